// Turns one instantiation of the GEMM kernel template into an entry of the host-side table.
#pragma once

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
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = Cfg::CG;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // Lets this launch be scheduled while the previous kernel of the stream winds down; the
  // kernel itself waits for that kernel's completion before it touches global memory.
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = a.serialize_programmatically ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, gemm_tf32_kernel<Cfg>, a.tmA, a.tmB, a.tmC, a.C, a.M, a.N, a.K,
                            a.ldc, a.tiles_m, a.tiles_n, a.chunk_kb, a.acc_kb, a.flags, a.status,
                            a.spin_limit, a.sk_tiles, a.sk_rounds, a.sk_ws, a.sk_flags, a.epoch,
                            a.peer, a.round_plan);
}

// The table's `mode` is the caller-visible one: 1 / 3 for fp32 operands (1xTF32 / 3xTF32),
// 16 for bf16 and 17 for fp16 operands.
template <int BN, int MODE, int CG, int LAYOUT = 0, int DT = 0, int STAGED = 0>
static KernelVariant make_variant() {
  using Cfg = GemmCfg<BN, MODE, CG, LAYOUT, DT, STAGED>;
  KernelVariant v;
  // In the skinny layout the kernel's 128-row side runs along N of the caller's problem.
  v.block_m = (LAYOUT == 2) ? BN : Cfg::TILE_M;
  v.block_n = (LAYOUT == 2) ? Cfg::TILE_M : BN;
  v.layout = LAYOUT;
  v.rstep = Cfg::BK;
  v.cta_group = CG;
  v.mode = (DT == 0) ? MODE : (DT == 1 ? 16 : 17);
  v.stages = Cfg::STAGES;
  v.smem_bytes = Cfg::SMEM_BYTES;
  v.tmem_cols = Cfg::TMEM_COLS;
  v.threads = Cfg::THREADS;
  v.staging_bytes = Cfg::STAGING_BYTES;
  v.gave_up_stage = STAGED;
  v.func = reinterpret_cast<const void*>(&gemm_tf32_kernel<Cfg>);
  v.launch = &launch_variant<Cfg>;
  return v;
}

}  // namespace rb200
