"""Roller rTile search: problem description, per-tile resource analysis and the ranking policies.

Public surface as in the reference's src/analyze.py: `Shape`, `MatmulConfig`, `TileDict`,
`Policy`, `compute_memory_traffic`, `get_roller_hints(matmul_config, arch, topk)`.

Two policies live here.

* `Policy` re-states the reference's heuristic (src/analyze.py:171-381) and, given the
  reference's `arch.CUDA()` model, returns the same hints in the same order. It is what the
  golden vectors under tests/golden/ pin.
* `BlackwellPolicy` ranks the rTiles that have an sm_100a kernel with a cost model of that
  kernel family (tensor-core rate, shared-memory and L2 feed rates, wave quantisation on 148
  SMs, HBM floor). `get_roller_hints` picks it when the device model is an `arch.B200`.
"""
from __future__ import annotations

import itertools
import math
from dataclasses import dataclass
from typing import Iterator, List, Optional

from .arch import B200, CUDA, TileDevice  # noqa: F401  (CUDA re-exported like the reference)
from .utils import coalesced_factor, coalesced_tensor_shape, get_all_factors


# --------------------------------------------------------------------------- problem description
@dataclass
class Shape:
    """A 2-D operand tile: S = spatial extent (rows of A / columns of B), R = reduce extent."""
    S: int
    R: int

    def to_list(self) -> List[int]:
        return [self.S, self.R]


@dataclass
class MatmulConfig:
    """C[M,N] = A[M,K] @ B[K,N] with `el_bits`-wide elements (src/analyze.py:26-49).

    The cost model treats both inputs as (spatial, reduce) with the reduce axis contiguous.
    """
    M: int
    N: int
    K: int
    el_bits: int

    def get_input_shapes(self):
        return Shape(S=self.M, R=self.K), Shape(S=self.N, R=self.K)

    def get_output_shape(self):
        return self.M, self.N

    @property
    def el_bytes(self) -> int:
        return (self.el_bits + 7) // 8

    @staticmethod
    def propagate_inputs(tile: List[int], rstep: int):
        return Shape(S=tile[0], R=rstep), Shape(S=tile[1], R=rstep)

    @staticmethod
    def propagate_outputs(tile: List[int]):
        return tile


def read_txn_elems(arch: TileDevice, el_bytes: int) -> int:
    """Elements per read transaction (src/analyze.py:52-54)."""
    return arch.transaction_size[1] // el_bytes


def write_txn_elems(arch: TileDevice, el_bytes: int) -> int:
    """Elements per global write transaction (src/analyze.py:57-59)."""
    return arch.transaction_size[0] // el_bytes


def compute_memory_traffic(output_tile: List[int], matmul_config: MatmulConfig,
                           arch: TileDevice) -> int:
    """Bytes one block moves for an output tile over the whole reduction: its A and B panels in
    read transactions plus its C tile in write transactions (src/analyze.py:62-81)."""
    eb = matmul_config.el_bytes
    rd, wr = read_txn_elems(arch, eb), write_txn_elems(arch, eb)
    panels = MatmulConfig.propagate_inputs(output_tile, matmul_config.K)
    elems = 0
    for panel, whole in zip(panels, matmul_config.get_input_shapes()):
        elems += coalesced_tensor_shape(panel.to_list(), whole.to_list(), rd)
    elems += coalesced_tensor_shape(output_tile, list(matmul_config.get_output_shape()), wr)
    return elems * eb


def _natural_size(n: int) -> str:
    """Binary-prefixed byte count for printing ("32.0 KiB")."""
    if n < 0:
        return str(n)
    if n < 1024:
        return f"{n} Byte" + ("" if n == 1 else "s")
    val = float(n)
    for unit in ("KiB", "MiB", "GiB", "TiB", "PiB"):
        val /= 1024.0
        if val < 1024.0:
            break
    return f"{val:.1f} {unit}"


# --------------------------------------------------------------------------- one candidate tile
class TileDict:
    """One rTile candidate: schedule knobs plus what the analysis derived for it
    (src/analyze.py:84-168). Callers read `block_tile`, `thread_tile`, `rstep`, `smem_cost` and
    `matmul_config` (src/roller.py:363-366,385,531-543); the Blackwell policy adds the fields
    listed in `BLACKWELL_FIELDS`."""

    BLACKWELL_FIELDS = ("cta_group", "stages", "mode", "tmem_cols", "est_us", "kernel", "layout")

    def __init__(self, block_tile: List[int], matmul_config: MatmulConfig, rstep: int) -> None:
        self.matmul_config = matmul_config
        self.block_tile = block_tile
        self.thread_tile: List[int] = []
        self.rstep = rstep
        self.traffic = -1
        self.smem_cost = -1
        self.block_per_SM = -1
        self.num_wave = -1
        self.grid_size = -1
        self.valid = True
        # Blackwell extras (None for hints of the generic policy)
        self.cta_group: Optional[int] = None
        self.stages: Optional[int] = None
        self.mode: Optional[int] = None
        self.tmem_cols: Optional[int] = None
        self.est_us: Optional[float] = None
        self.kernel: Optional[str] = None
        self.layout: int = 0   # 0 general tile, 2 skinny tile (tensor core works on C^T)

    def __hash__(self) -> int:
        return hash(tuple(self.block_tile + self.thread_tile))

    def __repr__(self) -> str:
        text = (f"TileDict(block_tile={self.block_tile}, thread_tile={self.thread_tile}, "
                f"rstep={self.rstep}, block traffic={_natural_size(self.traffic)}, "
                f"total traffic={_natural_size(self.traffic * self.grid_size)}, "
                f"smem_cost={_natural_size(self.smem_cost)}, block_per_SM={self.block_per_SM}, "
                f"num_wave={self.num_wave}, grid_size={self.grid_size}")
        if self.cta_group is not None:
            text += (f", cta_group={self.cta_group}, stages={self.stages}, mode={_mode_name(self.mode)}, "
                     f"tmem_cols={self.tmem_cols}, est={self.est_us:.1f} us")
        return text + ")"

    def clone(self) -> "TileDict":
        """Independent copy of the schedule (the problem description is shared)."""
        other = TileDict(list(self.block_tile), self.matmul_config, self.rstep)
        other.thread_tile = list(self.thread_tile)
        for name in ("traffic", "smem_cost", "block_per_SM", "num_wave", "grid_size", "valid",
                     *self.BLACKWELL_FIELDS):
            setattr(other, name, getattr(self, name))
        return other

    def infer_smem_usage(self, rstep: Optional[int] = None) -> int:
        """One pipeline stage: an rstep-deep slice of both operand panels."""
        step = self.rstep if rstep is None else rstep
        return sum(step * extent for extent in self.block_tile) * self.matmul_config.el_bytes

    @classmethod
    def from_block_tile(cls, block_tile: List[int], rstep: int, matmul_config: MatmulConfig,
                        arch: TileDevice) -> "TileDict":
        """Resource analysis of a block tile (src/analyze.py:125-168): shared memory and
        register feasibility, grid size, traffic, residency and wave count."""
        td = cls(block_tile, matmul_config, rstep)
        td.smem_cost = td.infer_smem_usage()
        if td.smem_cost > arch.smem_cap:
            td.valid = False
            return td
        # accumulators + operands, spread over a warp's worth of lanes
        regs = int(2 * math.prod(block_tile) * matmul_config.el_bytes / 32)
        if regs > arch.reg_cap:
            td.valid = False
            return td
        out = matmul_config.get_output_shape()
        td.grid_size = int(math.prod(-(-full // tile) for tile, full in zip(block_tile, out)))
        td.traffic = compute_memory_traffic(block_tile, matmul_config, arch)
        td.block_per_SM = min(arch.max_smem_usage // max(td.smem_cost, 1),
                              arch.reg_cap // max(regs, 1),
                              arch.sm_partition)
        resident = int(td.block_per_SM * arch.compute_max_core)
        td.num_wave = int(math.ceil(td.grid_size / resident))
        return td


# --------------------------------------------------------------------------- reference heuristic
class Policy:
    """The reference's default policy: minimise memory traffic, then maximise parallelism
    (src/analyze.py:171-381)."""

    def __init__(self, config: MatmulConfig, arch: TileDevice) -> None:
        self.arch = arch
        self.matmul_config = config

    # -- coalescing scores (src/analyze.py:181-201); larger is better
    def _coalesced_score(self, tile: List[int], rstep: int, mode: str = "sim") -> float:
        panels = MatmulConfig.propagate_inputs(tile, rstep)
        wholes = self.matmul_config.get_input_shapes()
        runs = [coalesced_factor(p.to_list(), w.to_list()) for p, w in zip(panels, wholes)]
        score = 0.0
        if mode == "sim":
            # closeness of each run length to one read transaction: 2ab / (a^2 + b^2)
            txn = read_txn_elems(self.arch, self.matmul_config.el_bytes)
            for run in runs:
                score += (2 * run * txn) / (run * run + txn * txn)
        else:
            for run in runs:
                score += run
        return score

    def get_reduce_step_candidates(self, rstep: int) -> List[int]:
        """Divisors of the reduce extent; for a prime above 64, powers of two below it
        (src/analyze.py:203-215)."""
        factors = get_all_factors(rstep)
        if len(factors) == 2 and rstep > 64:
            factors = [1]
            while factors[-1] * 2 < rstep:
                factors.append(factors[-1] * 2)
        return factors

    def _assign_reduce_step(self) -> int:
        candidates = self.get_reduce_step_candidates(self.matmul_config.K)
        return max(candidates, key=lambda step: self._coalesced_score([1, 1], step, "sim"))

    def get_block_tiles_candidates(self, init_tile: List[int], rstep: int) -> List[TileDict]:
        """Every (m, n) from divisors of M and N plus the small powers of two, analysed and
        ordered by (traffic + 1) * waves (src/analyze.py:223-255)."""
        axes = []
        for lo, extent in zip(init_tile, self.matmul_config.get_output_shape()):
            sizes = {f for f in get_all_factors(extent) if f >= lo}
            sizes.update(p for p in (2, 4, 8, 16, 32) if lo < p < extent)
            axes.append(sorted(sizes))
        tiles = []
        for m, n in itertools.product(*axes):
            td = TileDict.from_block_tile([m, n], rstep, self.matmul_config, self.arch)
            if td.valid:
                tiles.append(td)
        tiles.sort(key=lambda td: (td.traffic + 1) * td.num_wave)  # stable, like the reference
        return tiles

    def _expand_reduce_axis(self, td: TileDict) -> None:
        """Grow the reduce step to the best-coalesced divisor of K that is a multiple of the
        base step and still fits the per-block shared-memory share (src/analyze.py:257-277)."""
        limit = min(self.arch.max_smem_usage // td.block_per_SM, self.arch.smem_cap)
        fits = [s for s in self.get_reduce_step_candidates(self.matmul_config.K)
                if s % td.rstep == 0 and td.infer_smem_usage(s) <= limit]
        if not fits:
            fits = [td.rstep]
        td.rstep = max(fits, key=lambda s: self._coalesced_score(td.block_tile, s, "raw"))
        td.smem_cost = td.infer_smem_usage()

    def score_block_size(self, n: int):
        """(distance from one warp per sub-partition, padding waste); small is better
        (src/analyze.py:279-297)."""
        warps = (n + self.arch.warp_size - 1) // self.arch.warp_size
        balance = max(warps / self.arch.sm_partition, self.arch.sm_partition / warps)
        waste = (warps * self.arch.warp_size - n) / n
        return (balance, waste)

    def recommend_block_size(self, td: TileDict) -> List[int]:
        """Thread counts that divide the tile, at most 1024, best first (src/analyze.py:299-308)."""
        sizes = [f for f in get_all_factors(int(math.prod(td.block_tile))) if f <= 1024]
        return sorted(sizes, key=self.score_block_size)

    def assign_thread_tile(self, td: TileDict, topk: int = 1) -> Iterator[TileDict]:
        """Yield up to `topk` copies of `td`, one per recommended thread count, stopping at the
        first count whose thread tile does not fit the register budget (src/analyze.py:310-327)."""
        for block_size in self.recommend_block_size(td):
            hint = self._assign_thread_tile(td, block_size)
            if hint is None:
                return
            yield hint
            topk -= 1
            if topk == 0:
                return

    def _assign_thread_tile(self, td: TileDict, block_size: int) -> Optional[TileDict]:
        """Most square split of the per-thread element count, judged by operand reads over
        shared-memory bandwidth (src/analyze.py:329-365)."""
        per_thread = math.prod(td.block_tile) // block_size
        pairs = [[per_thread // i, i] for i in range(1, int(math.sqrt(per_thread)) + 1)
                 if per_thread % i == 0]
        K, smem_bw = self.matmul_config.K, self.arch.bandwidth[1]

        def read_cost(tile):
            cost = 0
            for extent in tile:
                cost += (extent * K) / smem_bw
            return cost

        best = min(pairs, key=read_cost)
        if int(math.prod(best) * self.matmul_config.el_bytes / 4) >= 256:
            return None
        td.thread_tile = best
        return td.clone()

    def emit_config(self, topk: int = 10) -> List[TileDict]:
        """Walk the ranked block tiles, two thread tiles each, until `topk` hints
        (src/analyze.py:367-381)."""
        rstep = self._assign_reduce_step()
        hints: List[TileDict] = []
        for td in self.get_block_tiles_candidates([1, 1], rstep):
            self._expand_reduce_axis(td)
            for hint in self.assign_thread_tile(td, 2):
                hints.append(hint)
                if len(hints) >= topk:
                    return hints
        return hints


# --------------------------------------------------------------------------- Blackwell policy
MODE_1XTF32 = 1     # fp32 operands, one TF32 product each
MODE_3XTF32 = 3     # fp32 operands, big/small split: three TF32 products, fp32-level accuracy
MODE_BF16 = 16      # bf16 operands (el_bits = 16), exact products, fp32 accumulation and C
MODE_F16 = 17       # fp16 operands (el_bits = 16), likewise


def _mode_name(mode) -> str:
    return {MODE_BF16: "bf16", MODE_F16: "fp16"}.get(mode, f"{mode}xTF32")


class BlackwellPolicy:
    """Ranks the compiled sm_100a rTiles for one problem.

    The reference ranks by (traffic + 1) * num_wave; the same two ideas -- bytes a block moves and
    how evenly blocks fill the machine -- appear here as terms of a time estimate:

      per k-block of `rstep` elements one CTA needs
        tensor  = block_m_per_cta * block_n * rstep * mode / macs_per_clk       clocks
        smem    = (bytes TMA writes + bytes the split warps read/write
                   + bytes the MMAs read) / smem_bytes_per_clk                   clocks
        l2      = raw operand bytes / l2_bytes_per_clk                            clocks
      a tile takes ceil(K / rstep) * max(tensor, smem, l2) clocks, a persistent worker runs
      ceil(tiles / workers) tiles (a fractional last wave when the library would use its
      stream-K schedule), and the whole GEMM cannot beat its HBM floor.
    Where the device model carries measured per-k-block times for a tile (`B200.kblock_us`),
    those replace the analytic per-k-block term.
    """

    def __init__(self, config: MatmulConfig, arch: B200, mode: Optional[int] = None) -> None:
        if config.el_bits == 32:
            mode = MODE_3XTF32 if mode is None else mode
            if mode not in (MODE_1XTF32, MODE_3XTF32):
                raise ValueError("fp32 operands: mode must be 1 (1xTF32) or 3 (3xTF32)")
        elif config.el_bits == 16:
            # the element width says 16-bit; whether that is bf16 or fp16 is the mode's business
            mode = MODE_BF16 if mode is None or mode in (MODE_1XTF32, MODE_3XTF32) else mode
            if mode not in (MODE_BF16, MODE_F16):
                raise ValueError("16-bit operands: mode must be 16 (bf16) or 17 (fp16)")
        else:
            raise ValueError("the sm_100a kernel family takes 32-bit or 16-bit operands "
                             "(el_bits must be 32 or 16)")
        self.matmul_config = config
        self.arch = arch
        self.mode = mode

    def _analyse(self, block_m: int, block_n: int, cta_group: int, stages: int,
                 layout: int = 0) -> TileDict:
        cfg, dev, mode = self.matmul_config, self.arch, self.mode
        eb = cfg.el_bytes
        sixteen = mode in (MODE_BF16, MODE_F16)
        rstep = dev.rstep * 4 // eb              # one 128-byte swizzle row of k
        # tensor-core products per operand product, and k per instruction
        products = 1 if sixteen else mode
        mma_k = dev.mma_k * 4 // eb
        macs_per_clk = dev.tf32_macs_per_clk_sm * (2 if sixteen else 1)
        td = TileDict([block_m, block_n], cfg, rstep)
        td.cta_group, td.stages, td.mode, td.layout = cta_group, stages, mode, layout
        if layout == 3:
            return self._analyse_cuda_core_tile(td, block_m, block_n)
        td.thread_tile = [1, 32]  # what one epilogue thread reads from TMEM at a time
        # the accumulator's columns are the tile's N side, or its M side in the skinny layout
        td.tmem_cols = 2 * (block_m if layout == 2 else block_n)
        rows_cta = block_m // cta_group          # A rows staged per CTA
        cols_cta = block_n // cta_group          # B columns staged per CTA
        raw = (rows_cta + cols_cta) * rstep * eb
        td.smem_cost = raw * (2 if mode == MODE_3XTF32 else 1)
        td.valid = (td.smem_cost * stages + 2048 <= dev.smem_cap and td.tmem_cols <= dev.tmem_columns)
        td.grid_size = (-(-cfg.M // block_m)) * (-(-cfg.N // block_n))
        td.traffic = compute_memory_traffic([block_m, block_n], cfg, dev)
        td.block_per_SM = 1
        workers = max(dev.compute_max_core // cta_group, 1)
        td.num_wave = -(-td.grid_size // workers)

        num_kb = -(-cfg.K // rstep)
        key = (block_m, block_n, cta_group) if layout == 0 else (block_m, block_n, cta_group, layout)
        measured = dev.kblock_us_16.get(key) if sixteen else dev.kblock_us.get(key)
        if measured is not None:
            kb_us = measured if sixteen else (measured[0] if mode == MODE_1XTF32 else measured[1])
        else:
            tensor_clk = rows_cta * block_n * rstep * products / macs_per_clk
            mma_reads = (rows_cta + cols_cta) * mma_k * eb * (rstep // mma_k) * products
            split_rw = 2 * raw if mode == MODE_3XTF32 else 0
            smem_clk = (raw + split_rw + mma_reads) / dev.smem_bytes_per_clk_sm
            l2_clk = raw / dev.l2_bytes_per_clk_sm
            kb_us = max(tensor_clk, smem_clk, l2_clk) / dev.sm_clock_mhz
        # Whole tiles go round-robin; leftover tiles are dealt out in pieces along K (stream-K)
        # when that shortens the schedule by 3 % or more after charging the partial-tile
        # exchange -- the same rule the library applies. 3xTF32 schedules in its 4-k-block
        # accumulation chunks and pays one of them (three when no whole tile follows); the
        # other modes schedule in units of 8 k-blocks and pay 24 k-blocks (72).
        full, left = divmod(td.grid_size, workers)
        waves = float(td.num_wave)
        if left:
            unit = 4 if mode == MODE_3XTF32 else min(8, num_kb)
            cpt = -(-num_kb // unit)
            exchange = (1 if mode == MODE_3XTF32 else -(-24 // unit)) * (1 if full >= 1 else 3)
            split = full * cpt + -(-left * cpt // workers) + exchange
            if cpt > 1 and (full + 1) * cpt - split >= 0.03 * (full + 1) * cpt:
                waves = split / cpt
        if layout == 2 and left:
            waves = full + left / workers   # the skinny layout always splits along K
        # launch, pipeline fill, last drain and the C stores of the final tile
        fixed_us = 8.0 + rows_cta * block_n * 4 / 32768.0
        worker_us = waves * num_kb * kb_us + fixed_us
        hbm_bytes = float(eb) * (cfg.M * cfg.K + cfg.K * cfg.N) + 4.0 * cfg.M * cfg.N
        hbm_us = hbm_bytes / (dev.hbm_gbs * 1e3) + 4.0
        td.est_us = max(worker_us, hbm_us)
        # operands whose rows are not 16-byte aligned are first copied into padded buffers
        # (one read + one write each, ahead of the GEMM)
        if cfg.K * eb % 16:
            td.est_us += 2.0 * eb * cfg.M * cfg.K / (dev.hbm_gbs * 1e3) * 1.5 + 3.0
        if cfg.N * eb % 16:
            td.est_us += 2.0 * eb * cfg.K * cfg.N / (dev.hbm_gbs * 1e3) * 1.5 + 3.0
        arith = {MODE_BF16: "bf16", MODE_F16: "f16"}.get(mode, f"{mode}x")
        td.kernel = (f"gemm_{'f16' if sixteen else 'tf32'}<{block_m}x{block_n}x{rstep},"
                     f"cg{cta_group},{arith}" + (",skinny>" if layout == 2 else ">"))
        return td

    def _analyse_cuda_core_tile(self, td: TileDict, block_m: int, block_n: int) -> TileDict:
        """The kernel that uses plain fp32 FMAs for a C of few rows (layout 3): a CTA per strip
        of `block_n` columns and range of K, one pass over B per `block_m` rows of C. Each byte
        of B feeds 16 FMAs, so a pass runs at whichever is slower, HBM or the FP32 lanes."""
        cfg, dev = self.matmul_config, self.arch
        td.thread_tile = [block_m, 4]       # partial sums one lane holds
        td.tmem_cols = 0
        td.smem_cost = 4 * block_m * 512    # one 512-k chunk of the A rows
        passes = -(-cfg.M // block_m)
        # one pass over B per 16 rows of C: only ranked for a C of few rows
        td.valid = cfg.el_bits == 32 and passes <= 4
        td.grid_size = passes * (-(-cfg.N // block_n))
        td.traffic = compute_memory_traffic([block_m, block_n], cfg, dev)
        td.block_per_SM = 2
        td.num_wave = -(-td.grid_size // (2 * dev.compute_max_core))
        hbm_us = 4.0 * passes * cfg.K * cfg.N / (dev.hbm_gbs * 1e3 * dev.cuda_core_hbm_frac)
        fma_us = (passes * block_m * cfg.K * cfg.N
                  / (dev.compute_max_core * 128 * dev.sm_clock_mhz * dev.cuda_core_fma_frac))
        td.est_us = max(hbm_us, fma_us) + 8.0
        td.kernel = f"skinny_fp32<{block_m}x{block_n},cuda cores>"
        return td

    def emit_config(self, topk: int = 10) -> List[TileDict]:
        sixteen = self.mode in (MODE_BF16, MODE_F16)
        tiles = [self._analyse(bm, bn, cg, s16 if sixteen else (s1 if self.mode == MODE_1XTF32 else s3),
                               layout)
                 for (bm, bn, cg, s1, s3, layout, s16) in self.arch.kernel_tiles
                 if (s16 > 0 if sixteen else (s1 if self.mode == MODE_1XTF32 else s3) > 0)]
        tiles = [td for td in tiles if td.valid]
        tiles.sort(key=lambda td: (td.est_us, td.traffic * td.grid_size))
        return tiles[:topk]


def get_roller_hints(matmul_config: MatmulConfig, arch: TileDevice, topk: int = 10,
                     mode: Optional[int] = None) -> List[TileDict]:
    """Top-k rTile hints, best first (src/analyze.py:384-387). `mode` only matters for a
    `B200` device model: 1 / 3 (1xTF32 / 3xTF32, default 3) for 32-bit operands, 16 / 17
    (bf16, the default, / fp16) for 16-bit operands."""
    if isinstance(arch, B200):
        return BlackwellPolicy(matmul_config, arch, mode).emit_config(topk)
    return Policy(matmul_config, arch).emit_config(topk)
