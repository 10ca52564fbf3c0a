// Instantiates the tcgen05 GEMM kernel family: one kernel per buildable rTile and mode.
// The reference compiles a kernel per hint at run time (src/roller.py:358-387); here the set
// is fixed at build time and the search is told which tiles exist.
#include "gemm_launch.h"
#include "gemm_tf32_sm100.cuh"

namespace rb200 {

template <class Cfg>
static cudaError_t launch_variant(const GemmArgs& a, int grid, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = Cfg::CG;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, gemm_tf32_kernel<Cfg>, a.tmA, a.tmB, a.C, a.M, a.N, a.K, a.ldc,
                            a.tiles_m, a.tiles_n, a.chunk_kb, a.flags, a.status, a.sk_tiles, a.sk_ws,
                            a.sk_flags, a.epoch);
}

template <int BN, int MODE, int CG, int LAYOUT = 0>
static KernelVariant make_variant() {
  using Cfg = GemmCfg<BN, MODE, CG, LAYOUT>;
  KernelVariant v;
  // In the skinny layout the kernel's 128-row side runs along N of the caller's problem.
  v.block_m = (LAYOUT == 2) ? BN : Cfg::TILE_M;
  v.block_n = (LAYOUT == 2) ? Cfg::TILE_M : BN;
  v.layout = LAYOUT;
  v.rstep = Cfg::BK;
  v.cta_group = CG;
  v.mode = MODE;
  v.stages = Cfg::STAGES;
  v.smem_bytes = Cfg::SMEM_BYTES;
  v.tmem_cols = Cfg::TMEM_COLS;
  v.threads = Cfg::THREADS;
  v.func = reinterpret_cast<const void*>(&gemm_tf32_kernel<Cfg>);
  v.launch = &launch_variant<Cfg>;
  return v;
}

static const KernelVariant* table(int* n) {
  static const KernelVariant kTable[] = {
      make_variant<256, 1, 2>(), make_variant<256, 3, 2>(),
      make_variant<128, 1, 2>(), make_variant<128, 3, 2>(),
      make_variant<64, 1, 2>(),  make_variant<64, 3, 2>(),
      make_variant<256, 1, 1>(), make_variant<256, 3, 1>(),
      make_variant<128, 1, 1>(), make_variant<128, 3, 1>(),
      make_variant<64, 1, 1>(),  make_variant<64, 3, 1>(),
      // B given transposed (Bt[N,K]): both operands K-major
      make_variant<256, 1, 2, 1>(), make_variant<256, 3, 2, 1>(),
      make_variant<128, 1, 1, 1>(), make_variant<128, 3, 1, 1>(),
      make_variant<64, 1, 1, 1>(),  make_variant<64, 3, 1, 1>(),
      // skinny C (few rows): roles swapped, tile = 64 or 32 rows of C x 128 columns
      make_variant<64, 1, 1, 2>(),  make_variant<64, 3, 1, 2>(),
      make_variant<32, 1, 1, 2>(),  make_variant<32, 3, 1, 2>(),
  };
  *n = static_cast<int>(sizeof(kTable) / sizeof(kTable[0]));
  return kTable;
}

int variant_count() {
  int n;
  table(&n);
  return n;
}

const KernelVariant& variant_at(int idx) {
  int n;
  return table(&n)[idx];
}

const KernelVariant* find_variant(int block_m, int block_n, int rstep, int cta_group, int mode,
                                  int layout) {
  int n;
  const KernelVariant* t = table(&n);
  for (int i = 0; i < n; ++i) {
    if (t[i].block_m == block_m && t[i].block_n == block_n && t[i].rstep == rstep &&
        t[i].cta_group == cta_group && t[i].mode == mode && t[i].layout == layout)
      return &t[i];
  }
  return nullptr;
}

}  // namespace rb200
