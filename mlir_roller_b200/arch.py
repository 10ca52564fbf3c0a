"""Device models for the rTile search.

Mirrors the reference's `arch` module (src/arch.py): `TileDevice` is the generic description the
search reads, `CUDA` reproduces the reference's A100-like numbers field for field (it is kept so
that the search can be checked against the reference's own output), and `B200` is the model the
sm_100a kernel family is ranked with.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Tuple


def _pair(a: int, b: int):
    return field(default_factory=lambda: [a, b])


@dataclass
class TileDevice:
    """What the search needs to know about a device (field names as in src/arch.py:15-34)."""

    reg_cap: int = 0                 # 32-bit registers per SM
    smem_cap: int = 0                # shared memory one block may use, bytes
    compute_max_core: int = 0        # number of SMs
    warp_size: int = 0
    sm_partition: int = 0            # sub-partitions (warp schedulers) per SM
    max_smem_usage: int = 0          # shared memory per SM that resident blocks may share
    platform: str = "unknown"
    compute_capability: str = "unknown"
    l2_cache_size_bytes: int = 0
    transaction_size: List[int] = _pair(0, 0)   # [global write, global read] bytes
    bandwidth: List[int] = _pair(0, 0)          # [global, shared] relative bandwidths

    def get_avaliable_tensorintrin_shapes(self):
        raise NotImplementedError()


@dataclass
class CUDA(TileDevice):
    """The reference's only device model (src/arch.py:40-61): an A100-class part."""

    platform: str = "CUDA"
    smem_cap: int = 64 * 1024
    compute_max_core: int = 108
    warp_size: int = 32
    reg_cap: int = 65536
    sm_partition: int = 4
    transaction_size: List[int] = _pair(32, 128)
    bandwidth: List[int] = _pair(750, 12080)
    max_smem_usage: int = field(init=False)

    def __post_init__(self):
        # two blocks' worth of the per-block cap may be resident per SM
        self.max_smem_usage = 2 * self.smem_cap


# rTiles for which libroller_b200 carries a compiled kernel:
# (block_m, block_n, cta_group, stages_1x, stages_3x, layout, stages_16); stages_16 is the
# pipeline depth of the tile's kernel for 16-bit operands (0 = none). Layout 0 is the general tile;
# layout 2 is the "skinny" tile for a C with few rows (the tensor core works on C^T, so the
# narrow side, block_m, runs along M). Kept in step with the library by a test that compares
# the table against roller_b200_kernel_desc().
B200_KERNEL_TILES: Tuple[Tuple[int, int, int, int, int, int, int], ...] = (
    (256, 256, 2, 7, 3, 0, 7),
    (256, 128, 2, 8, 4, 0, 8),
    (256, 64, 2, 8, 5, 0, 0),
    (128, 256, 1, 4, 2, 0, 4),
    (128, 128, 1, 7, 3, 0, 7),
    (128, 64, 1, 8, 4, 0, 8),
    (64, 128, 1, 8, 4, 2, 8),
    (32, 128, 1, 8, 5, 2, 8),
    # layout 3: the CUDA-core kernel (plain fp32 FMAs) for a C of at most 16 rows per pass;
    # it has a 3xTF32-class form only (fp32-exact products), hence 0 stages for the others
    (16, 256, 1, 0, 1, 3, 0),
)


# Measured steady-state cost of one 32-deep k-block on one worker (CTA or CTA pair), in
# microseconds, per compiled rTile: (block_m, block_n, cta_group) -> (1xTF32, 3xTF32).
# Taken on a B200 at 4096 x 8192 x 16384 (clock ~1.7 GHz under the power cap). The 256x256 pair
# tile runs near the tensor rate; narrower tiles are held back by shared-memory bandwidth and,
# in 3xTF32, by the split pass competing with fewer pipeline stages.
B200_KBLOCK_US = {
    (256, 256, 2): (0.410, 1.114),
    (256, 128, 2): (0.320, 0.803),
    (256, 64, 2): (0.275, 0.690),
    (128, 256, 1): (0.515, 1.521),
    (128, 128, 1): (0.321, 0.927),
    (128, 64, 1): (0.278, 0.702),
    # skinny tiles, keyed with their layout; measured at 16 x 16384 x 16384, where they stream B
    # at 5.7 TB/s (1xTF32) / 3.6 TB/s (3xTF32)
    (32, 128, 1, 2): (0.39, 0.63),
    (64, 128, 1, 2): (0.40, 0.66),
}


# The same for the 16-bit kernels (bf16 / fp16 operands): one k-block is 64 deep, i.e. the same
# 128 bytes per operand row and the same number of tensor-core clocks as a 1xTF32 k-block.
# Measured at 8192^3 and 4096^3 in bf16; the narrow and skinny entries are the 1xTF32 figures
# scaled by the ratio seen on the measured tiles (1.13).
B200_KBLOCK_US_16 = {
    (256, 256, 2): 0.445,
    (256, 128, 2): 0.364,
    (128, 256, 1): 0.575,
    (128, 128, 1): 0.362,
    (128, 64, 1): 0.314,
    (32, 128, 1, 2): 0.44,
    (64, 128, 1, 2): 0.45,
}


@dataclass
class B200(TileDevice):
    """NVIDIA B200 (sm_100a): 148 SMs, 227 KiB shared memory per block, tensor memory.

    The generic fields keep their meaning so that the reference's resource checks still read
    sensibly; the Blackwell-specific fields below drive the cost model of
    `analyze.BlackwellPolicy`. Bandwidth and peak figures default to values measured on this
    class of device and can be overwritten (e.g. from `roller_b200_device_info`).
    """

    platform: str = "CUDA"
    compute_capability: str = "100a"
    smem_cap: int = 227 * 1024          # opt-in maximum per block
    compute_max_core: int = 148
    warp_size: int = 32
    reg_cap: int = 65536
    sm_partition: int = 4
    l2_cache_size_bytes: int = 126 * 1024 * 1024
    transaction_size: List[int] = _pair(32, 128)
    bandwidth: List[int] = _pair(6532, 12080 * 4)
    max_smem_usage: int = 228 * 1024    # one persistent block per SM

    # --- Blackwell additions
    tmem_columns: int = 512             # 128 lanes x 512 columns x 32 bit per SM
    rstep: int = 32                     # one 128-byte swizzle row of fp32
    mma_k: int = 8                      # k per tcgen05.mma kind::tf32
    tf32_macs_per_clk_sm: int = 2048    # dense TF32 multiply-accumulates per clock per SM
    smem_bytes_per_clk_sm: int = 128
    l2_bytes_per_clk_sm: float = 64.0   # sustained L2 -> SM fill rate per SM
    sm_clock_mhz: float = 1700.0        # typical clock under tensor load (1965 boost)
    hbm_gbs: float = 6532.0             # measured copy bandwidth
    tf32_tflops: float = 790.0          # measured dense TF32 rate (cuBLAS, 8192^3)
    kernel_tiles: Tuple[Tuple[int, int, int, int, int, int, int], ...] = B200_KERNEL_TILES
    kblock_us: dict = field(default_factory=lambda: dict(B200_KBLOCK_US))
    kblock_us_16: dict = field(default_factory=lambda: dict(B200_KBLOCK_US_16))
    bf16_tflops: float = 1621.6         # measured dense bf16 rate (cuBLAS, 8192^3, burst)
    # the CUDA-core kernel for a C of few rows: fraction of the HBM copy rate it streams B at,
    # and fraction of the FP32 lanes' issue rate its FMAs reach (fitted to measurements)
    cuda_core_hbm_frac: float = 0.75
    cuda_core_fma_frac: float = 0.42

    @classmethod
    def from_device(cls, dev: int = 0) -> "B200":
        """Fill the generic fields from the library's device query."""
        from . import _lib
        info = _lib.device_info(dev)
        model = cls()
        model.compute_max_core = info.sm_count
        model.smem_cap = info.smem_per_block_optin
        model.max_smem_usage = info.smem_per_sm
        model.reg_cap = info.regs_per_sm
        model.l2_cache_size_bytes = info.l2_bytes
        model.tmem_columns = info.tmem_columns
        model.compute_capability = f"{info.cc_major}{info.cc_minor}a"
        model.kernel_tiles = tuple(
            (kt.block_m, kt.block_n, kt.cta_group, kt.stages_1x, kt.stages_3x, kt.layout,
             kt.stages_16)
            for kt in _lib.kernel_tiles())
        return model
