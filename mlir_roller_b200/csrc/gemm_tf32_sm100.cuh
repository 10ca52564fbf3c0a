// fp32 GEMM C[M,N] = A[M,K] @ B[K,N] (all row-major) on the sm_100a tensor cores.
//
// This kernel family replaces the per-hint generated `gemm_kernel` of the reference
// (schedule: src/roller.py:93-342, payload linalg.matmul: src/roller.py:47-68). One
// instantiation exists per rTile the search may emit: block tile (128*CG) x BN, reduce step 32.
//
// The same template also serves 16-bit operands (bf16 / fp16 A and B, fp32 C): tcgen05.mma
// kind::f16, reduce step 64, one MMA per 16 k; everything else below applies unchanged.
//
// Arithmetic: tcgen05.mma kind::tf32 with fp32 accumulation in TMEM.
//   MODE 1 ("1xTF32"): one MMA per k-step. The tensor core reads only the top 19 bits of each
//          32-bit word (truncation, measured on B200), so the host encodes the tensor maps of
//          this mode with the TFLOAT32 data type: the TMA unit then rounds every element to the
//          nearest TF32 value while copying it into shared memory.
//   MODE 3 ("3xTF32"): each operand x is used as big(x) = the raw word (its low 13 bits are not
//          read) and small(x) = x - trunc19(x), computed exactly in fp32 by the split warps and
//          rounded to 19 bits; per k-step three MMAs small*big + big*small + big*big go into
//          the same accumulator.
// The TMEM accumulator rounds toward zero on every MMA, which on B200 shows up as an error that
// grows linearly with the number of MMAs chained into one accumulator (1.7e-5 of max|C| at
// K = 2048 in 3xTF32). The reduction is therefore cut into chunks of `chunk_kb` k-blocks: each
// chunk is accumulated in TMEM from zero, then drained by the epilogue warps into fp32
// registers with round-to-nearest adds while the next chunk runs in the other TMEM buffer.
//
// Pipeline (one persistent CTA, or CTA pair when CG == 2, per SM; 16 warps):
//   warp 0        TMA producer: A box 128x32 (K-major, 128B swizzle), B boxes 32x32
//                 (N contiguous, 128B swizzle on 32-byte chunks) into a STAGES-deep ring
//   warp 1        MMA issuer (one thread, leader CTA only) + TMEM allocation
//   warps 4..11   accumulate/epilogue: warp w owns TMEM lanes 32*(w%4).. and one half of the
//                 tile's columns; sums chunk results in registers, stores C with tail predicates
//   warps 12..15  split warps (MODE 3) write the small parts next to the raw tiles and tell the
//                 leader CTA's barrier that the stage is ready
// With a CTA pair in MODE 1 both CTAs' TMA loads report straight to the leader's barrier.
// Ragged M/N/K need no special main loop: TMA zero-fills out-of-range elements.
//
// Operand layouts (template parameter LAYOUT). Each MMA operand tile is either "K-major" (its
// rows are contiguous along k in global memory: one TMA box of ROWS x 32, 128-byte swizzle) or
// "MN-major" (contiguous along m or n: boxes of 32 x 32, 128-byte swizzle on 32-byte chunks).
//   0  A[M,K] row-major (K-major), B[K,N] row-major (MN-major): the reference's layout.
//   1  A as above, B given transposed as Bt[N,K] row-major (K-major).
//   2  "skinny": for a C with few rows the roles are swapped -- the tensor core computes
//      C^T = B^T A^T, so the 128-row side of the MMA runs along N, the narrow side (32 or 64)
//      along M, nothing but real data is staged, and the epilogue writes C transposed (which
//      makes its stores coalesced). The kernel then sees M' = N, N' = M, A' = B (MN-major),
//      B' = A (K-major).
//
// Work distribution. Tiles are handed to the persistent workers (CTAs or CTA pairs) round-robin.
// When the tile count does not divide by the worker count, the last, partly filled wave would
// leave SMs idle, so the first `sk_tiles` tiles are instead cut along K into chunk-sized units
// that are dealt evenly to all workers ("stream-K"). A worker that computes only part of a
// tile's reduction writes its partial sums to its slot of a global scratch area and raises a
// flag; the worker that holds the end of the tile's reduction adds the slots of the others and
// stores C. Every worker runs its stream-K units first (the piece it must publish before the
// piece it must complete), then its whole tiles, so these waits are short; they are bounded
// like every other wait in the kernel.
//
// "Progressive" schedule (sk_rounds > 1, every tile cut along K). The tiles are taken in
// `sk_rounds` groups of consecutive tiles; the whole grid works on one group at a time, each
// worker on a few k-chunks of it, so finished tiles leave the kernel at a steady rate from
// early on instead of all together at the end. That is what a consumer on the far side of a
// link wants (the multi-GPU driver stores C straight into another GPU's memory): the transfer
// then runs underneath the rest of the computation. A worker reuses its scratch slot from
// round to round, so it waits (bounded) for the slot's reader before it publishes again.
//
// Output path. By default the accumulate warps store C themselves. With kFlagTmaStore (kernels
// that have a staging area, Cfg::STAGING_BYTES > 0) each warp writes 32 x 32 pieces of its
// part of the tile into shared memory and hands them to the TMA unit
// (cp.async.bulk.tensor store), which drains them to global memory on its own: the warps are
// back at the next tile's accumulation at once, however slowly the destination (a peer GPU
// behind NVLink) takes the data.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "gemm_launch.h"
#include "ptx_sm100.cuh"


namespace rb200 {

// One operand tile of ROWS (m or n) x 128 bytes of k (32 fp32 or 64 16-bit elements) whose
// global rows run along k.
template <int ROWS>
struct OperandK {
  static constexpr int BYTES = ROWS * 128;
  static constexpr uint32_t MAJOR = 0;   // instruction-descriptor major bit: K
  static constexpr uint64_t KK_STEP = 2; // one MMA (32 bytes of k) further along a row, >> 4
  template <bool PAIR>
  static __device__ __forceinline__ void load(uint32_t dst, const CUtensorMap* tm, uint32_t bar,
                                              int row0, int k0) {
    if constexpr (PAIR) tma_load_2d_pair(dst, tm, bar, k0, row0);
    else tma_load_2d(dst, tm, bar, k0, row0);
  }
  // rows of 128 B, 8-row swizzle atoms 1024 B apart
  static __device__ __forceinline__ uint64_t desc(uint32_t addr) {
    return make_smem_desc(addr, 16, 1024, kLayoutSw128);
  }
};

// One operand tile of ROWS (m or n) x BK (k) whose global rows run along m/n, for elements of
// EB bytes. It is staged as boxes of BK rows (one k each) of 128 bytes (32 fp32 or 64 16-bit
// m/n values).
template <int ROWS, int EB = 4>
struct OperandMN {
  static constexpr int BOX_MN = 128 / EB;           // m/n values per box row
  static constexpr int BOX_K = 128 / EB;            // k rows per box (= the reduce step)
  static constexpr int BOXES = ROWS / BOX_MN;
  static constexpr int BOX_BYTES = BOX_K * 128;
  static constexpr int BYTES = BOXES * BOX_BYTES;
  static constexpr uint32_t MAJOR = 1;    // MN
  // one MMA further: 8 (fp32) or 16 (16-bit) rows of a box = 1024 or 2048 B, >> 4
  static constexpr uint64_t KK_STEP = (EB == 4) ? 64 : 128;
  static_assert(ROWS % BOX_MN == 0, "whole boxes");
  template <bool PAIR>
  static __device__ __forceinline__ void load(uint32_t dst, const CUtensorMap* tm, uint32_t bar,
                                              int row0, int k0) {
#pragma unroll
    for (int j = 0; j < BOXES; ++j) {
      if constexpr (PAIR) tma_load_2d_pair(dst + j * BOX_BYTES, tm, bar, row0 + j * BOX_MN, k0);
      else tma_load_2d(dst + j * BOX_BYTES, tm, bar, row0 + j * BOX_MN, k0);
    }
  }
  // fp32: 4-row swizzle atoms (32-byte chunks) 512 B apart along k. 16-bit: the ordinary
  // 128-byte swizzle, 8-row atoms 1024 B apart along k. Either way the next box_mn values of
  // m/n are one whole box further.
  static __device__ __forceinline__ uint64_t desc(uint32_t addr) {
    if constexpr (EB == 4) return make_smem_desc(addr, BOX_BYTES, 512, kLayoutSw128Base32);
    else return make_smem_desc(addr, BOX_BYTES, 1024, kLayoutSw128);
  }
};

// DT_: operand element type. 0 = fp32 (tensor-core kind tf32), 1 = bf16, 2 = fp16 (kind f16).
// STAGED_: 1 = a ring that would fill shared memory gives up one stage to make room for the
// staging area of the TMA-store output path (measured on B200, 256 x 256 pair tile, 1xTF32 and
// bf16: 8-14 % faster at 2048^3, even at K = 4096, 2-5 % slower at K = 8192; so both forms of
// such a kernel exist and the host picks by K).
template <int BN_, int MODE_, int CG_, int LAYOUT_ = 0, int DT_ = 0, int STAGED_ = 0>
struct GemmCfg {
  static constexpr int BN = BN_;      // tile columns (of the CTA pair when CG == 2)
  static constexpr int MODE = MODE_;  // 1 or 3 tensor-core products per operand product
  static constexpr int CG = CG_;      // CTAs cooperating on one tile (tcgen05 cta_group)
  static constexpr int LAYOUT = LAYOUT_;
  static constexpr int DT = DT_;
  static constexpr int EB = (DT == 0) ? 4 : 2;  // bytes per operand element
  static constexpr bool TRANSPOSE_C = (LAYOUT == 2);
  static constexpr int BM = 128;      // tile rows held by one CTA
  static constexpr int BK = 128 / EB; // reduce step: one 128-byte swizzle row of k
  static constexpr int MMA_K = 32 / EB;  // k per tensor-core instruction
  static constexpr int BNL = BN / CG; // B columns staged by one CTA
  using AOp = typename std::conditional<LAYOUT == 2, OperandMN<BM, EB>, OperandK<BM>>::type;
  using BOp = typename std::conditional<LAYOUT == 0, OperandMN<BNL, EB>, OperandK<BNL>>::type;
  static constexpr int A_BYTES = AOp::BYTES;
  static constexpr int B_BYTES = BOp::BYTES;
  static constexpr int RAW_BYTES = (A_BYTES + B_BYTES + 1023) / 1024 * 1024;
  // 3xTF32 keeps the split-off small parts next to the raw tile, in the same stage. (A second,
  // short ring for the small parts with a deeper landing ring was measured on the skinny
  // tiles, where it should matter most: 16 x 8192 x 8192 went from 84 to 117 us.)
  static constexpr int STAGE_BYTES = (MODE == 3 ? 2 : 1) * RAW_BYTES;
  static constexpr int CTRL_BYTES = 256;
  static constexpr int SMEM_LIMIT = 232448;  // 227 KiB opt-in maximum per CTA
  static constexpr int STAGES_FIT = (SMEM_LIMIT - 1024 - CTRL_BYTES) / STAGE_BYTES;
  // Staging area of the TMA-store output path: one 32 x 32 fp32 box (128-byte swizzle) per
  // accumulate warp. Kernels without the area only have the plain store path (C written
  // transposed never uses it).
  static constexpr int STAGING_WANTED = 8 * 4096;
  static constexpr int STAGES_BESIDE_STAGING =
      (SMEM_LIMIT - 1024 - CTRL_BYTES - STAGING_WANTED) / STAGE_BYTES;
  static constexpr bool GIVES_UP_A_STAGE = STAGED_ != 0;
  static_assert(!GIVES_UP_A_STAGE || (LAYOUT_ != 2 && STAGES_FIT <= 8 &&
                                      STAGES_BESIDE_STAGING == STAGES_FIT - 1),
                "only a ring that fills shared memory has a stage to give up");
  static constexpr int STAGES = GIVES_UP_A_STAGE ? STAGES_BESIDE_STAGING
                                                 : (STAGES_FIT > 8 ? 8 : STAGES_FIT);
  static constexpr int STAGING_BYTES =
      (LAYOUT_ != 2 &&
       SMEM_LIMIT - 1024 - CTRL_BYTES - STAGES * STAGE_BYTES >= STAGING_WANTED)
          ? STAGING_WANTED : 0;
  static constexpr int SMEM_BYTES =
      STAGES * STAGE_BYTES + STAGING_BYTES + CTRL_BYTES + 1024;
  static constexpr int ACC_STAGES = 2;
  static constexpr int TMEM_COLS = ACC_STAGES * BN;
  static constexpr bool HAS_XFORM = (MODE == 3);
  static constexpr int XFORM_WARPS = 4;
  static constexpr int FIRST_EPI_WARP = 4;
  static constexpr int EPI_WARPS = 8;
  static constexpr int FIRST_XFORM_WARP = 12;
  static constexpr int THREADS = 512;
  static constexpr int EPI_COLS = BN / 2;  // accumulator columns one epilogue thread owns
  static constexpr int MMA_M = BM * CG;
  static constexpr int TILE_M = BM * CG;
  // Register rebalancing between warpgroups (only the widest tile needs it): 512 threads get
  // 128 registers each at launch; the control and split warpgroups give some back so that the
  // two accumulate warpgroups can hold 128 accumulators per thread.
  static constexpr bool REBALANCE = (EPI_COLS > 64);
  static constexpr int REGS_CTRL = 64, REGS_XFORM = 80, REGS_EPI = 184;

  static_assert(BN % (32 * CG) == 0, "each CTA stages whole 32-column boxes of B");
  static_assert(DT == 0 || MODE == 1, "split precision exists for fp32 operands only");
  static_assert(EPI_COLS % 16 == 0, "epilogue threads read whole 16-column slabs");
  static_assert(EPI_COLS % 32 == 0 || EPI_COLS == 16, "C is stored in pieces of 32 (or 16) columns");
  static_assert(TMEM_COLS == 64 || TMEM_COLS == 128 || TMEM_COLS == 256 || TMEM_COLS == 512,
                "power of two");
  static_assert(LAYOUT != 2 || CG == 1, "the skinny layout runs on single CTAs");
  static_assert(STAGES >= 2, "need at least a double buffer");
  static_assert(RAW_BYTES % 1024 == 0, "swizzle atoms must stay 1024-byte aligned");
  static_assert(4 * (REGS_CTRL + REGS_XFORM + 2 * REGS_EPI) * 32 <= 65536, "register file");
};

// Tile order: walk the output in panels of 8 tile-rows so that concurrently running CTAs
// share A row panels and B column panels in L2 (the reference swizzles thread blocks with
// panel width 8 for the same reason, src/roller.py:334-339).
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& mb, int& nb) {
  constexpr int kPanel = 8;
  const int per_panel = kPanel * tiles_n;
  const int panel = t / per_panel;
  const int first_m = panel * kPanel;
  const int rows = min(tiles_m - first_m, kPanel);
  const int r = t - panel * per_panel;
  mb = first_m + r % rows;
  nb = r / rows;
}

// small(x) = x - trunc19(x), then rounded to nearest on the 19-bit grid the tensor core reads.
__device__ __forceinline__ uint32_t split_small(uint32_t xb) {
  const float x = __uint_as_float(xb);
  const float big = __uint_as_float(xb & 0xFFFFE000u);
  // Three instructions per element: the split warps sit on the critical path of the narrower
  // tiles. An infinite x gives inf - inf = nan here, so infinities surface as nan in 3xTF32.
  return __float_as_uint(x - big) + 0x1000u;
}

// fp32 <-> the 16-bit operand type of a kernel (DT 1 = bf16, 2 = fp16), round to nearest even.
template <int DT>
__device__ __forceinline__ uint32_t to_16bit(float x) {
  if constexpr (DT == 1) return __bfloat16_as_ushort(__float2bfloat16_rn(x));
  else return __half_as_ushort(__float2half_rn(x));
}
template <int DT>
__device__ __forceinline__ float from_16bit(uint32_t b) {
  if constexpr (DT == 1) return __uint_as_float(b << 16);
  else return __half2float(__ushort_as_half(static_cast<unsigned short>(b)));
}
template <int DT>
__device__ __forceinline__ uint32_t pack_16bit(float lo, float hi) {
  return to_16bit<DT>(lo) | (to_16bit<DT>(hi) << 16);
}

template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}

// One unit of work for all roles of a worker: k-blocks [kb0, kb1) of tile `tile`.
struct Segment {
  int tile;
  int kb0, kb1;
  bool final;  // holds the end of the tile's reduction: adds the other workers' partials, stores C
  int round;   // round of the schedule the segment belongs to (0 for whole tiles)
  int pos;     // the worker's position in that round
};

// Static schedule shared by the producer, split, MMA and epilogue roles (each walks its own copy).
//
// The first `sk_tiles` tiles are cut into units of `chunk_kb` k-blocks and worked through in
// `rounds` rounds: round r owns tiles [tile_begin[r], tile_begin[r + 1]) (RoundPlan, made by
// the host; no tile straddles two rounds), and its units, in tile order, are dealt out in
// contiguous runs to the `workers` positions of the round. With rounds == 1 that is the plain
// stream-K deal. The remaining tiles follow whole, round-robin. Rounds need not be equally
// large: when C leaves over a link while the computation goes on, rounds that shrink (or grow)
// geometrically keep the link busy from early on and leave little to send after the last one.
// From one round to the next the workers change places (worker w plays position
// (w + round * rot) mod workers of the round): without the rotation the same few workers would
// end up completing a tile -- and paying for the exchange of partial sums -- in every round
// while all others wait for them.
// All of it is 32-bit arithmetic (the host only enables the split when units < 2^31): a 64-bit
// division is a subroutine call on the device.
struct RoundShape {
  int base;          // first unit of the round
  int tiles;         // tiles the round owns
  uint32_t q, rem;   // units of the round / workers, and the remainder
};

struct Schedule {
  int num_tiles, workers, worker, num_kb, chunk_kb, cpt, sk_tiles, rounds;
  const RoundPlan* plan;
  int round;             // round whose units are being consumed
  int rot;               // positions the workers move on from one round to the next
  int pos;               // this worker's position in the current round
  int u_begin, u_end;    // this worker's units of the current round, consumed from the end
  int dp_next;           // next whole tile

  __device__ Schedule(int num_tiles_, int workers_, int worker_, int num_kb_, int chunk_kb_,
                      int sk_tiles_, int rounds_, const RoundPlan* plan_)
      : num_tiles(num_tiles_), workers(workers_), worker(worker_), num_kb(num_kb_),
        chunk_kb(chunk_kb_), sk_tiles(sk_tiles_), rounds(rounds_), plan(plan_), round(0) {
    cpt = (num_kb + chunk_kb - 1) / chunk_kb;
    rot = rounds > 1 ? (workers * 3) / 8 + 1 : 0;
    pos = worker;
    const RoundShape rs = shape(0);
    u_begin = unit_begin(rs, worker);
    u_end = unit_begin(rs, worker + 1);
    dp_next = sk_tiles + worker;
  }
  __device__ RoundShape shape(int r) const {
    RoundShape rs;
    const int t0 = rounds > 1 ? static_cast<int>(plan->tile_begin[r]) : 0;
    const int t1 = rounds > 1 ? static_cast<int>(plan->tile_begin[r + 1]) : sk_tiles;
    rs.base = t0 * cpt;
    rs.tiles = t1 - t0;
    const uint32_t units = static_cast<uint32_t>(rs.tiles) * static_cast<uint32_t>(cpt);
    rs.q = units / static_cast<uint32_t>(workers);
    rs.rem = units - rs.q * static_cast<uint32_t>(workers);
    return rs;
  }
  // Worker at position `p` of round `r`.
  __device__ int worker_at(int p, int r) const {
    int w = (p - r * rot) % workers;
    return w < 0 ? w + workers : w;
  }
  // First unit of position p (0 .. workers) of a round:
  // base + floor(units * p / workers) = base + q * p + floor(rem * p / workers).
  __device__ int unit_begin(const RoundShape& rs, int p) const {
    const uint32_t up = static_cast<uint32_t>(p);
    return rs.base + static_cast<int>(rs.q * up + rs.rem * up / static_cast<uint32_t>(workers));
  }
  __device__ bool next(Segment& s) {
    while (u_end <= u_begin && round + 1 < rounds) {
      ++round;
      pos = (worker + round * rot) % workers;
      const RoundShape rs = shape(round);
      u_begin = unit_begin(rs, pos);
      u_end = unit_begin(rs, pos + 1);
    }
    if (u_end > u_begin) {
      const int tile = (u_end - 1) / cpt;
      const int t0 = tile * cpt;
      const int sb = u_begin > t0 ? u_begin : t0;
      s.tile = tile;
      s.kb0 = (sb - t0) * chunk_kb;
      s.kb1 = min((u_end - t0) * chunk_kb, num_kb);
      s.final = (u_end - t0 == cpt);
      s.round = round;
      s.pos = pos;
      u_end = sb;
      return true;
    }
    if (dp_next < num_tiles) {
      s.tile = dp_next;
      s.kb0 = 0;
      s.kb1 = num_kb;
      s.final = true;
      s.round = 0;
      s.pos = worker;
      dp_next += workers;
      return true;
    }
    return false;
  }
};

// System scope: the other party is another GPU of the node (or its copy engine).
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Barrier among the 256 accumulate/epilogue threads only (hardware barrier 1).
__device__ __forceinline__ void epi_bar_sync() {
  asm volatile("bar.sync 1, 256;" ::: "memory");
}
// The same barrier carrying a vote: true for every thread when any of the 256 passed `mine`.
// The accumulate warps use it wherever they must agree on giving up: a warp that left on its
// own would leave the others waiting at the next barrier for ever.
__device__ __forceinline__ bool epi_bar_any(bool mine) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.or.pred p, 1, 256, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(out)
      : "r"(static_cast<uint32_t>(mine))
      : "memory");
  return out != 0;
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
gemm_tf32_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, float* __restrict__ C, int M, int N, int K,
                 long long ldc, int tiles_m, int tiles_n, int chunk_kb, int acc_kb, int flags,
                 uint32_t* status, long long spin_limit, int sk_tiles, int sk_rounds, float* sk_ws,
                 uint32_t* sk_flags, uint32_t epoch, const PeerSync peer,
                 const __grid_constant__ RoundPlan round_plan) {
  // chunk_kb: the unit of the stream-K schedule (a tile's reduction is dealt out in pieces of
  // that many k-blocks); acc_kb: how many k-blocks accumulate in TMEM before the accumulate
  // warps drain them into registers. 3xTF32 uses the same value for both; the modes whose
  // accuracy does not ask for frequent drains schedule in small units and drain rarely.
  constexpr int BN = Cfg::BN, BK = Cfg::BK, CG = Cfg::CG, STAGES = Cfg::STAGES;

  extern __shared__ uint8_t smem_dyn[];
  const uint32_t smem_dyn_addr = smem_addr(smem_dyn);
  const uint32_t smem_base = (smem_dyn_addr + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_dyn + (smem_base - smem_dyn_addr);

  const uint32_t staging = smem_base + STAGES * Cfg::STAGE_BYTES;   // 1024-byte aligned
  const uint32_t ctrl = staging + Cfg::STAGING_BYTES;
  auto full_bar = [&](int s) { return ctrl + 8u * s; };         // TMA bytes landed (per CTA)
  auto ready_bar = [&](int s) { return ctrl + 64u + 8u * s; };  // stage usable by MMA (leader)
  auto empty_bar = [&](int s) { return ctrl + 128u + 8u * s; }; // MMAs done reading (per CTA)
  auto tmem_full_bar = [&](int a) { return ctrl + 192u + 8u * a; };
  auto tmem_empty_bar = [&](int a) { return ctrl + 208u + 8u * a; };
  const uint32_t tmem_slot = ctrl + 224u;
  const uint32_t mma_done_bar = ctrl + 240u;   // every MMA of this launch has completed
  const WaitCtx wc{status, spin_limit};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = (CG == 2) ? cluster_ctarank() : 0u;
  const bool is_leader = (cta_rank == 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(ready_bar(s), CG * Cfg::XFORM_WARPS);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < Cfg::ACC_STAGES; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), CG * Cfg::EPI_WARPS);
    }
    mbar_init(mma_done_bar, 1);
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc<CG>(tmem_slot, Cfg::TMEM_COLS);
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if constexpr (Cfg::STAGING_BYTES > 0) {
      if (flags & kFlagTmaStore) tma_prefetch_desc(&tmC);
    }
  }
  // The next kernel of the stream may be scheduled from now on (its CTAs take SMs as this
  // grid's CTAs leave them and wait below); nothing above touched global memory.
  grid_launch_dependents();
  tcgen05_fence_before_sync();
  if constexpr (CG == 2) cluster_sync(); else __syncthreads();
  tcgen05_fence_after_sync();
  // Everything from here on reads operands, scratch and status that the previous kernel of
  // the stream may have written, and writes C.
  grid_dependency_wait();

  uint32_t tmem_base;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

  const int num_kb = (K + BK - 1) / BK;
  Schedule sched(tiles_m * tiles_n, static_cast<int>(gridDim.x) / CG,
                 static_cast<int>(blockIdx.x) / CG, num_kb, chunk_kb, sk_tiles, sk_rounds,
                 &round_plan);
  Segment sg;

  if (warp < Cfg::FIRST_EPI_WARP) {
    if constexpr (Cfg::REBALANCE) setmaxnreg_dec<Cfg::REGS_CTRL>();
    if (warp == 0 && lane == 0) {
      // ---------------------------------------------------------- TMA producer
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      while (ok && sched.next(sg)) {
        int mb, nb;
        tile_coords(sg.tile, tiles_m, tiles_n, mb, nb);
        const int m0 = (mb * CG + static_cast<int>(cta_rank)) * Cfg::BM;
        const int n0 = nb * BN + static_cast<int>(cta_rank) * Cfg::BNL;
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          if (!mbar_wait(empty_bar(s), ph ^ 1u, wc, kDevTimeoutEmpty)) { ok = false; break; }
          const uint32_t a_dst = smem_base + s * Cfg::STAGE_BYTES;
          const uint32_t b_dst = a_dst + Cfg::A_BYTES;
          if constexpr (CG == 2 && !Cfg::HAS_XFORM) {
            // The leader's barrier counts the bytes of both CTAs; only the leader arms it.
            if (is_leader) mbar_expect_tx(full_bar(s), 2 * (Cfg::A_BYTES + Cfg::B_BYTES));
            const uint32_t bar = map_to_cta(full_bar(s), 0);
            Cfg::AOp::template load<true>(a_dst, &tmA, bar, m0, kb * BK);
            Cfg::BOp::template load<true>(b_dst, &tmB, bar, n0, kb * BK);
          } else {
            mbar_expect_tx(full_bar(s), Cfg::A_BYTES + Cfg::B_BYTES);
            Cfg::AOp::template load<false>(a_dst, &tmA, full_bar(s), m0, kb * BK);
            Cfg::BOp::template load<false>(b_dst, &tmB, full_bar(s), n0, kb * BK);
          }
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
      // Tail: the MMA issuer's last releases must land in this CTA before it may exit.
      for (int i = 0; i < STAGES && ok; ++i) {
        ok = mbar_wait(empty_bar(s), ph ^ 1u, wc, kDevTimeoutTail);
        if (++s == STAGES) { s = 0; ph ^= 1u; }
      }
      // ... and so must the arrival that closes the MMA issuer's work (sent to both CTAs).
      mbar_wait_drain(mma_done_bar, 0u, spin_limit);
    } else if (warp == 1 && lane == 0 && is_leader) {
      // ---------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc =
          Cfg::DT == 0 ? make_idesc_tf32(Cfg::MMA_M, BN, Cfg::AOp::MAJOR, Cfg::BOp::MAJOR)
                       : make_idesc_f16(Cfg::MMA_M, BN, Cfg::AOp::MAJOR, Cfg::BOp::MAJOR,
                                        Cfg::DT == 1 ? 1u : 0u);
      constexpr uint64_t a_step = Cfg::AOp::KK_STEP, b_step = Cfg::BOp::KK_STEP;
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
      while (ok && sched.next(sg)) {
        for (int kb0 = sg.kb0; kb0 < sg.kb1 && ok; kb0 += acc_kb) {
          const int kb1 = min(kb0 + acc_kb, sg.kb1);
          if (!mbar_wait(tmem_empty_bar(acc), acc_ph ^ 1u, wc, kDevTimeoutTmemEmpty)) {
            ok = false;
            break;
          }
          tcgen05_fence_after_sync();
          const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
          for (int kb = kb0; kb < kb1; ++kb) {
            const uint32_t wait_bar = Cfg::HAS_XFORM ? ready_bar(s) : full_bar(s);
            if (!mbar_wait(wait_bar, ph, wc, kDevTimeoutReady)) { ok = false; break; }
            tcgen05_fence_after_sync();
            const uint32_t stage = smem_base + s * Cfg::STAGE_BYTES;
            const uint64_t a_raw = Cfg::AOp::desc(stage);
            const uint64_t b_raw = Cfg::BOp::desc(stage + Cfg::A_BYTES);
            // One MMA consumes 32 bytes of k (8 fp32 or 16 16-bit elements) of both tiles.
            if constexpr (Cfg::MODE == 3) {
              const uint64_t a_sml = Cfg::AOp::desc(stage + Cfg::RAW_BYTES);
              const uint64_t b_sml = Cfg::BOp::desc(stage + Cfg::RAW_BYTES + Cfg::A_BYTES);
              // Correction terms first: they are 2^-11 of the main term, so adding them while
              // the accumulator is still small costs the least rounding.
#pragma unroll
              for (int kk = 0; kk < BK / 8; ++kk) {
                umma_tf32<CG>(d_tmem, a_sml + kk * a_step, b_raw + kk * b_step, idesc,
                              (kb != kb0 || kk != 0) ? 1u : 0u);
                umma_tf32<CG>(d_tmem, a_raw + kk * a_step, b_sml + kk * b_step, idesc, 1u);
              }
#pragma unroll
              for (int kk = 0; kk < BK / 8; ++kk)
                umma_tf32<CG>(d_tmem, a_raw + kk * a_step, b_raw + kk * b_step, idesc, 1u);
            } else if constexpr (Cfg::DT == 0) {
#pragma unroll
              for (int kk = 0; kk < BK / 8; ++kk)
                umma_tf32<CG>(d_tmem, a_raw + kk * a_step, b_raw + kk * b_step, idesc,
                              (kb != kb0 || kk != 0) ? 1u : 0u);
            } else {
#pragma unroll
              for (int kk = 0; kk < BK / Cfg::MMA_K; ++kk)
                umma_f16<CG>(d_tmem, a_raw + kk * a_step, b_raw + kk * b_step, idesc,
                             (kb != kb0 || kk != 0) ? 1u : 0u);
            }
            umma_commit<CG>(empty_bar(s));
            if (++s == STAGES) { s = 0; ph ^= 1u; }
          }
          if (ok) umma_commit<CG>(tmem_full_bar(acc));
          acc ^= 1;
          if (acc == 0) acc_ph ^= 1u;
        }
      }
      // Whatever was issued must have completed before tensor and shared memory are given
      // up, also when the loop above was left early. (Not cut short by a recorded error.)
      umma_commit<CG>(mma_done_bar);
      mbar_wait_drain(mma_done_bar, 0u, spin_limit);
    }
  } else if (warp < Cfg::FIRST_XFORM_WARP) {
    // ------------------------------------------------------------ accumulate + epilogue
    if constexpr (Cfg::REBALANCE) setmaxnreg_inc<Cfg::REGS_EPI>();
    constexpr int COLS = Cfg::EPI_COLS;
    constexpr int PIECE = COLS < 32 ? COLS : 32;   // columns of row-major C stored at a time
    const int quarter = warp & 3;  // TMEM lanes a warp may read: 32 * (warp id mod 4)
    const int half = (warp - Cfg::FIRST_EPI_WARP) >> 2;
    const int et = static_cast<int>(threadIdx.x) - Cfg::FIRST_EPI_WARP * 32;  // 0..255
    const bool accumulate = (flags & kFlagAccumulate) != 0;
    const bool vec_store = (flags & kFlagVecStore) != 0;
    // 16-bit kernels can also write C in their operand type (C then points to 16-bit elements)
    const bool c16 = Cfg::DT != 0 && (flags & kFlagC16) != 0;
    const bool tma_store = Cfg::STAGING_BYTES > 0 && (flags & kFlagTmaStore) != 0;
    const bool smem_store = Cfg::STAGING_BYTES > 0 && !tma_store && (flags & kFlagSmemStore) != 0;
    // With partial tiles in play the 256 threads meet at barriers, so they must also leave
    // together: every decision to give up is then taken by a vote at such a barrier.
    const bool sk_active = sk_tiles > 0;
    // Stream-K scratch: one slot of 128 x BN floats per CTA; thread `et` owns every 256th float4.
    constexpr size_t kSlotFloats = static_cast<size_t>(Cfg::BM) * BN;
    int acc = 0;
    uint32_t acc_ph = 0;
    bool ok = true;
    float sum[COLS];

    // ---- cooperative completion of shared tiles (kFlagCoopFixup; needs the staging area).
    // Every worker holding part of a tile publishes its partial sums, and the tile is then
    // completed by all of them together: each takes some of the 32-column boxes, adds that
    // slice of everybody's partial in a fixed order and hands it to the TMA unit. The cost per
    // worker no longer grows with the number of workers sharing a tile, and nobody waits for
    // one worker that adds everything alone. A worker publishes up to two partials per round
    // (the head of one tile, the tail of another), notes them here, and completes its slices
    // when it moves on to the next round, while its MMAs already run ahead.
    const bool coop = Cfg::STAGING_BYTES > 0 && (flags & kFlagCoopFixup) != 0 && tma_store;
    constexpr int NB = COLS / 32 > 0 ? COLS / 32 : 1;   // boxes per warp and tile
    int pend_tile0 = 0, pend_tile1 = 0, pend_pos0 = 0, pend_pos1 = 0;   // (scalars: no local array)
    int npend = 0, pend_round = 0;
    // ---- hand-shake with another GPU (kFlagPeerSync): C is that GPU's memory, which it may
    // still be reading for the previous step. Nothing is stored before its "go" has arrived;
    // the wait sits in front of a warp's first store, so it costs nothing while the first
    // tiles are being computed. A wait that runs out records kDevTimeoutPeer and lets the
    // stores go ahead: the launch is reported as failed and its C is not to be used.
    bool go_pending = Cfg::STAGING_BYTES > 0 && (flags & kFlagPeerSync) != 0 && peer.go_flag != nullptr;
    auto await_go = [&]() {     // (lane 0 of the warp, which issues its stores)
      const long long t0 = clock64();
      uint32_t spins = 0;
      while (static_cast<int32_t>(ld_acquire_sys(peer.go_flag) - peer.go_value) < 0) {
        if ((++spins & 15u) == 0 && clock64() - t0 > spin_limit) {
          atomicCAS(status, kDevOk, kDevTimeoutPeer);
          break;
        }
      }
      go_pending = false;
    };
    uint32_t* const sk_reads = sk_flags + 4 * gridDim.x;   // one reader count per slot
    // slot of worker w's partial of a round: two per round (see `which_of`), two rounds alive
    auto coop_slot = [&](int w, int round, int which) {
      return (static_cast<size_t>(w) * CG + cta_rank) * 4 + static_cast<size_t>((round & 1) * 2 + which);
    };
    // which of a position's two partials of a round belongs to tile t: the one holding the
    // position's last unit is published first (0), the other one (1) second
    auto which_of = [&](const RoundShape& rs, int p, int t) {
      return ((sched.unit_begin(rs, p + 1) - 1) / sched.cpt == t) ? 0 : 1;
    };
    auto flush_pending = [&]() -> bool {
      for (int e = 0; e < npend; ++e) {
        const int T = e ? pend_tile1 : pend_tile0, pos = e ? pend_pos1 : pend_pos0, round = pend_round;
        const uint32_t tag = (epoch << 6) | static_cast<uint32_t>(round);
        const RoundShape rs = sched.shape(round);
        const int u0 = T * sched.cpt, u1 = u0 + sched.cpt;
        int p_first = pos, p_last = pos;
        while (p_first > 0 && sched.unit_begin(rs, p_first) > u0) --p_first;
        while (p_last < sched.workers - 1 && sched.unit_begin(rs, p_last + 1) < u1) ++p_last;
        int P = 0, my_idx = 0;
        for (int p = p_first; p <= p_last; ++p) {
          if (sched.unit_begin(rs, p + 1) == sched.unit_begin(rs, p)) continue;   // no units
          if (p < pos) ++my_idx;
          ++P;
        }
        const int R = P < NB ? P : NB;          // workers that complete a share of the tile
        if (my_idx >= R) continue;              // (uniform over the CTA) not one of them
        // wait for every partial of the tile: thread i watches position p_first + i
        const int mine = p_first + et;
        const bool watching = mine <= p_last &&
                              sched.unit_begin(rs, mine + 1) != sched.unit_begin(rs, mine);
        uint32_t* my_watch = nullptr;
        bool failed = false;
        if (watching) {
          my_watch = sk_flags + coop_slot(sched.worker_at(mine, round), round, which_of(rs, mine, T));
          const long long t0 = clock64();
          uint32_t spins = 0;
          while (ld_acquire_gpu(my_watch) != tag) {
            if ((++spins & 63u) == 0) {
              if (*reinterpret_cast<volatile uint32_t*>(status) != kDevOk) { failed = true; break; }
              if (clock64() - t0 > spin_limit) {
                atomicCAS(status, kDevOk, kDevTimeoutFixup);
                failed = true;
                break;
              }
            }
          }
        }
        if (epi_bar_any(failed)) return false;
        int mb, nb;
        tile_coords(T, tiles_m, tiles_n, mb, nb);
        const int row0 = (mb * CG + static_cast<int>(cta_rank)) * Cfg::BM + quarter * 32;
        const uint32_t box = staging + static_cast<uint32_t>(warp - Cfg::FIRST_EPI_WARP) * 4096u;
        for (int c = my_idx; c < NB; c += R) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.0f;
          for (int p = p_first; p <= p_last; ++p) {
            if (sched.unit_begin(rs, p + 1) == sched.unit_begin(rs, p)) continue;
            const float4* slot = reinterpret_cast<const float4*>(
                sk_ws + coop_slot(sched.worker_at(p, round), round, which_of(rs, p, T)) * kSlotFloats);
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
              const float4 q = __ldcg(slot + (8 * c + jj) * 256 + et);
              v[4 * jj] += q.x; v[4 * jj + 1] += q.y; v[4 * jj + 2] += q.z; v[4 * jj + 3] += q.w;
            }
          }
          const int col0 = nb * BN + half * COLS + c * 32;
          if (row0 < M && col0 < N) {
            if (lane == 0) bulk_wait_read_all();   // the box's previous contents have left
            __syncwarp();
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
              const uint32_t at = box + static_cast<uint32_t>(lane) * 128u +
                                  (static_cast<uint32_t>(jj ^ (lane & 7)) << 4);
              asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(at), "f"(v[4 * jj]),
                           "f"(v[4 * jj + 1]), "f"(v[4 * jj + 2]), "f"(v[4 * jj + 3])
                           : "memory");
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              if (go_pending) await_go();
              tma_store_2d(&tmC, box, col0, row0);
              bulk_commit_group();
            }
          }
        }
        // Every thread has read what it needs. Count this reader on each partial's slot; the
        // last of the R readers hands the slot back to its owner.
        epi_bar_sync();
        if (watching) {
          uint32_t* reads = sk_reads + (my_watch - sk_flags);
          if (atomicAdd(reads, 1u) == static_cast<uint32_t>(R - 1)) {
            *reinterpret_cast<volatile uint32_t*>(reads) = 0u;
            __threadfence();
            st_release_gpu(my_watch, 0u);
          }
        }
      }
      npend = 0;
      return true;
    };

    int rs_round = -1;
    RoundShape rs_cur = {0, 0, 0u, 0u};
    bool coop_round = false;
    while (ok && sched.next(sg)) {
      if constexpr (Cfg::STAGING_BYTES > 0) {
        if (coop && npend > 0 && sg.round != pend_round) {
          if (!flush_pending()) { ok = false; break; }
        }
      }
      if (sk_active && sg.round != rs_round) {
        rs_round = sg.round;
        rs_cur = sched.shape(sg.round);
        // Whether the round's shared tiles are completed by all their workers together is
        // decided per round, the same way by everybody: it pays where a tile is shared by
        // three workers or more (measured: a tenth dearer with one or two, a third to a half
        // cheaper beyond four).
        coop_round = coop && sched.workers >= 3 * rs_cur.tiles;
      }
      int mb, nb;
      tile_coords(sg.tile, tiles_m, tiles_n, mb, nb);
      const int row = (mb * CG + static_cast<int>(cta_rank)) * Cfg::BM + quarter * 32 + lane;
      const int n0 = nb * BN + half * COLS;
#pragma unroll
      for (int j = 0; j < COLS; ++j) sum[j] = 0.0f;
      for (int kb0 = sg.kb0; kb0 < sg.kb1; kb0 += acc_kb) {
        // (a warp gives up as a whole: the tensor-memory loads below need all 32 lanes)
        if (!__all_sync(0xffffffffu, mbar_wait(tmem_full_bar(acc), acc_ph, wc, kDevTimeoutTmemFull))) {
          ok = false;
          break;
        }
        tcgen05_fence_after_sync();
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                               static_cast<uint32_t>(acc * BN + half * COLS);
#pragma unroll
        for (int c = 0; c < COLS / 16; ++c) {
          uint32_t v[16];
          tmem_ld_32x16(t_row + static_cast<uint32_t>(c * 16), v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) sum[c * 16 + j] += __uint_as_float(v[j]);
        }
        tcgen05_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if constexpr (CG == 2) mbar_arrive_cluster(tmem_empty_bar(acc), 0);
          else mbar_arrive(tmem_empty_bar(acc));
        }
        acc ^= 1;
        if (acc == 0) acc_ph ^= 1u;
      }
      if (sk_active) {
        if (epi_bar_any(!ok)) { ok = false; break; }
      } else if (!ok) {
        break;
      }

      if constexpr (Cfg::STAGING_BYTES > 0) {
        if (coop_round && !(sg.kb0 == 0 && sg.final)) {
          // part of a shared tile: publish it and note it; it is completed in flush_pending
          const size_t slot_i = coop_slot(sched.worker, sg.round, which_of(rs_cur, sg.pos, sg.tile));
          uint32_t* my_flag = sk_flags + slot_i;
          if (sg.round > 1) {
            // the slot still holds the partial of two rounds ago until its readers are done
            bool failed = false;
            if (et == 0) {
              const long long t0 = clock64();
              uint32_t spins = 0;
              while (ld_acquire_gpu(my_flag) != 0u) {
                if ((++spins & 63u) == 0) {
                  if (*reinterpret_cast<volatile uint32_t*>(status) != kDevOk) { failed = true; break; }
                  if (clock64() - t0 > spin_limit) {
                    atomicCAS(status, kDevOk, kDevTimeoutSlot);
                    failed = true;
                    break;
                  }
                }
              }
            }
            if (epi_bar_any(failed)) { ok = false; break; }
          }
          float4* slot = reinterpret_cast<float4*>(sk_ws + slot_i * kSlotFloats);
#pragma unroll
          for (int j = 0; j < COLS / 4; ++j)
            slot[j * 256 + et] = make_float4(sum[4 * j], sum[4 * j + 1], sum[4 * j + 2], sum[4 * j + 3]);
          epi_bar_sync();
          if (et == 0 && !(flags & kFlagDropPublish))
            st_release_gpu(my_flag, (epoch << 6) | static_cast<uint32_t>(sg.round));
          if (npend == 0) { pend_tile0 = sg.tile; pend_pos0 = sg.pos; }
          else { pend_tile1 = sg.tile; pend_pos1 = sg.pos; }
          pend_round = sg.round;
          ++npend;
          continue;
        }
      }
      // Flags carry the launch and the round, so a slot's reader never takes one round's
      // partial sums for another's; zero means "slot free". Here a worker publishes at most once
      // per round, into the first of the round's two slots (the same numbering as the
      // cooperative form, which may be in use in other rounds of the launch); the slots
      // alternate from round to round, so a worker only ever waits for a reader that is two
      // rounds behind.
      const uint32_t tag = (epoch << 6) | static_cast<uint32_t>(sg.round);
      auto slot_index = [&](int w) {
        return (static_cast<size_t>(w) * CG + cta_rank) * 4 + static_cast<size_t>((sg.round & 1) * 2);
      };
      if (!sg.final) {
        // Publish this worker's partial sums of the tile, then raise its flag.
        uint32_t* my_flag = sk_flags + slot_index(sched.worker);
        if (sg.round > 1) {
          // The slot still holds the partial of two rounds ago until its reader hands it back.
          bool failed = false;
          if (et == 0) {
            const long long t0 = clock64();
            uint32_t spins = 0;
            while (ld_acquire_gpu(my_flag) != 0u) {
              if ((++spins & 63u) == 0) {
                if (*reinterpret_cast<volatile uint32_t*>(status) != kDevOk) { failed = true; break; }
                if (clock64() - t0 > spin_limit) {
                  atomicCAS(status, kDevOk, kDevTimeoutSlot);
                  failed = true;
                  break;
                }
              }
            }
          }
          if (epi_bar_any(failed)) { ok = false; break; }
        }
        float4* slot = reinterpret_cast<float4*>(sk_ws + slot_index(sched.worker) * kSlotFloats);
#pragma unroll
        for (int j = 0; j < COLS / 4; ++j)
          slot[j * 256 + et] = make_float4(sum[4 * j], sum[4 * j + 1], sum[4 * j + 2], sum[4 * j + 3]);
        // The barrier orders all 256 threads' stores before thread 0's release store below, whose
        // gpu scope then covers them for whoever acquires the flag.
        epi_bar_sync();
        // (a launch made for a test of the bounded waits leaves the flag down)
        if (et == 0 && !(flags & kFlagDropPublish)) st_release_gpu(my_flag, tag);
        continue;
      }
      if (sg.kb0 > 0) {
        // Add the partial sums of the workers that computed the earlier parts of this tile:
        // the positions before this one in the same round, down to the one that started the
        // tile. First every partial is awaited at once (thread i watches the flag of the i-th
        // position back), then they are added in a fixed order -- the result does not depend on
        // who arrived first -- and finally all slots are handed back together.
        const int tile_u0 = sg.tile * sched.cpt;
        int p_first = sg.pos - 1;
        while (p_first > 0 && sched.unit_begin(rs_cur, p_first) > tile_u0) --p_first;
        const int mine = sg.pos - 1 - et;     // the position this thread watches, if any
        const bool watching = mine >= p_first &&
                              sched.unit_begin(rs_cur, mine + 1) != sched.unit_begin(rs_cur, mine);
        bool failed = false;
        if (watching) {
          const uint32_t* flag = sk_flags + slot_index(sched.worker_at(mine, sg.round));
          const long long t0 = clock64();
          uint32_t spins = 0;
          while (ld_acquire_gpu(flag) != tag) {
            if ((++spins & 63u) == 0) {
              if (*reinterpret_cast<volatile uint32_t*>(status) != kDevOk) { failed = true; break; }
              if (clock64() - t0 > spin_limit) {
                atomicCAS(status, kDevOk, kDevTimeoutFixup);
                failed = true;
                break;
              }
            }
          }
        }
        if (epi_bar_any(failed)) { ok = false; break; }
        for (int p = sg.pos - 1; p >= p_first; --p) {
          // A position with no units in this round published nothing.
          if (sched.unit_begin(rs_cur, p + 1) == sched.unit_begin(rs_cur, p)) continue;
          const float4* slot = reinterpret_cast<const float4*>(
              sk_ws + slot_index(sched.worker_at(p, sg.round)) * kSlotFloats);
#pragma unroll
          for (int j = 0; j < COLS / 4; ++j) {
            const float4 q = __ldcg(slot + j * 256 + et);
            sum[4 * j] += q.x; sum[4 * j + 1] += q.y; sum[4 * j + 2] += q.z; sum[4 * j + 3] += q.w;
          }
        }
        // Hand the slots back (each partial has exactly one reader): with the flag at zero
        // again its owner may publish into the slot two rounds on, and a replay of this very
        // launch -- a captured CUDA graph re-issues the same epoch -- cannot take the old
        // contents for new ones.
        epi_bar_sync();
        if (watching)
          st_release_gpu(sk_flags + slot_index(sched.worker_at(mine, sg.round)), 0u);
      }
      if constexpr (Cfg::STAGING_BYTES > 0) {
        if (tma_store) {
          // Hand the tile to the TMA unit in 32 x 32 pieces through this warp's staging box.
          // Box rows are 128 bytes; the 16-byte chunk c of row r sits at chunk (c ^ (r & 7)),
          // the 128-byte swizzle the tensor map of C is encoded with (and the order in which a
          // warp's 32 lanes hit every bank exactly once per four rows).
          const uint32_t box = staging + static_cast<uint32_t>(warp - Cfg::FIRST_EPI_WARP) * 4096u;
          const int row0 = (mb * CG + static_cast<int>(cta_rank)) * Cfg::BM + quarter * 32;
          if (row0 < M) {
#pragma unroll
            for (int c = 0; c < COLS / 32; ++c) {
              const int col0 = n0 + c * 32;
              if (col0 >= N) break;
              if (lane == 0) bulk_wait_read_all();   // the box's previous contents have left
              __syncwarp();
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const uint32_t at = box + static_cast<uint32_t>(lane) * 128u +
                                    (static_cast<uint32_t>(j ^ (lane & 7)) << 4);
                asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(at),
                             "f"(sum[c * 32 + 4 * j]), "f"(sum[c * 32 + 4 * j + 1]),
                             "f"(sum[c * 32 + 4 * j + 2]), "f"(sum[c * 32 + 4 * j + 3])
                             : "memory");
              }
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                if (go_pending) await_go();
                tma_store_2d(&tmC, box, col0, row0);
                bulk_commit_group();
              }
            }
          }
          continue;
        }
        if (smem_store) {
          // C's rows start anywhere (an odd leading dimension), so neither TMA nor 128-bit
          // stores apply, and a lane storing its own row would touch 32 different rows per
          // instruction. The 32 x 32 pieces go through this warp's staging box instead and
          // are read back row by row: lane l then holds column l, and one store writes 128
          // consecutive bytes of a row of C.
          const uint32_t box = staging + static_cast<uint32_t>(warp - Cfg::FIRST_EPI_WARP) * 4096u;
          const int row0 = (mb * CG + static_cast<int>(cta_rank)) * Cfg::BM + quarter * 32;
          if (row0 < M) {
#pragma unroll
            for (int c = 0; c < COLS / 32; ++c) {
              const int col0 = n0 + c * 32;
              if (col0 >= N) break;
              __syncwarp();     // the previous piece has been read back by every lane
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const uint32_t at = box + static_cast<uint32_t>(lane) * 128u +
                                    (static_cast<uint32_t>(j ^ (lane & 7)) << 4);
                asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(at),
                             "f"(sum[c * 32 + 4 * j]), "f"(sum[c * 32 + 4 * j + 1]),
                             "f"(sum[c * 32 + 4 * j + 2]), "f"(sum[c * 32 + 4 * j + 3])
                             : "memory");
              }
              __syncwarp();
              const int col = col0 + lane;
              const int rows_here = min(32, M - row0);
              float* dst = C + static_cast<size_t>(row0) * static_cast<size_t>(ldc) + col;
              if (col < N) {
#pragma unroll 8
                for (int r = 0; r < rows_here; ++r) {
                  const uint32_t at = box + static_cast<uint32_t>(r) * 128u +
                                      (static_cast<uint32_t>((lane >> 2) ^ (r & 7)) << 4) +
                                      (static_cast<uint32_t>(lane & 3) << 2);
                  float v;
                  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(at) : "memory");
                  if (accumulate) v += *dst;
                  *dst = v;
                  dst += ldc;
                }
              }
            }
          }
          continue;
        }
      }
      if constexpr (Cfg::TRANSPOSE_C) {
        // The kernel computed C^T: element (row, col) of its tile is C[col][row], so for one
        // register the 32 lanes of a warp write 32 consecutive floats of a row of C.
        if (row < M) {
#pragma unroll
          for (int j = 0; j < COLS; ++j) {
            const int col = n0 + j;
            if (col < N) {
              const size_t at = static_cast<size_t>(col) * static_cast<size_t>(ldc) + row;
              float o = sum[j];
              if constexpr (Cfg::DT != 0) {
                if (c16) {
                  unsigned short* dst = reinterpret_cast<unsigned short*>(C) + at;
                  if (accumulate) o += from_16bit<Cfg::DT>(*dst);
                  *dst = static_cast<unsigned short>(to_16bit<Cfg::DT>(o));
                  continue;
                }
              }
              float* dst = C + at;
              if (accumulate) o += *dst;
              *dst = o;
            }
          }
        }
      } else if (row < M && c16) {
        if constexpr (Cfg::DT != 0) {
          unsigned short* crow =
              reinterpret_cast<unsigned short*>(C) + static_cast<size_t>(row) * static_cast<size_t>(ldc);
#pragma unroll
          for (int c = 0; c < COLS / PIECE; ++c) {
            const int col0 = n0 + c * PIECE;
            if (col0 >= N) break;
            unsigned short* dst = crow + col0;
            if (vec_store && col0 + PIECE <= N) {
              uint4* dst4 = reinterpret_cast<uint4*>(dst);   // 8 elements per 128-bit store
#pragma unroll
              for (int j = 0; j < PIECE / 8; ++j) {
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = sum[c * PIECE + 8 * j + e];
                if (accumulate) {
                  const uint4 old = dst4[j];
                  const uint32_t w[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    v[2 * e] += from_16bit<Cfg::DT>(w[e] & 0xFFFFu);
                    v[2 * e + 1] += from_16bit<Cfg::DT>(w[e] >> 16);
                  }
                }
                dst4[j] = make_uint4(pack_16bit<Cfg::DT>(v[0], v[1]), pack_16bit<Cfg::DT>(v[2], v[3]),
                                     pack_16bit<Cfg::DT>(v[4], v[5]), pack_16bit<Cfg::DT>(v[6], v[7]));
              }
            } else {
#pragma unroll
              for (int j = 0; j < PIECE; ++j) {
                if (col0 + j < N) {
                  float o = sum[c * PIECE + j];
                  if (accumulate) o += from_16bit<Cfg::DT>(dst[j]);
                  dst[j] = static_cast<unsigned short>(to_16bit<Cfg::DT>(o));
                }
              }
            }
          }
        }
      } else if (row < M) {
        float* crow = C + static_cast<size_t>(row) * static_cast<size_t>(ldc);
#pragma unroll
        for (int c = 0; c < COLS / PIECE; ++c) {
          const int col0 = n0 + c * PIECE;
          if (col0 >= N) break;
          float* dst = crow + col0;
          if (vec_store && col0 + PIECE <= N) {
            float4* dst4 = reinterpret_cast<float4*>(dst);
#pragma unroll
            for (int j = 0; j < PIECE / 4; ++j) {
              float4 o = make_float4(sum[c * PIECE + 4 * j], sum[c * PIECE + 4 * j + 1],
                                     sum[c * PIECE + 4 * j + 2], sum[c * PIECE + 4 * j + 3]);
              if (accumulate) {
                const float4 old = dst4[j];
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              dst4[j] = o;
            }
          } else {
#pragma unroll
            for (int j = 0; j < PIECE; ++j) {
              if (col0 + j < N) {
                float o = sum[c * PIECE + j];
                if (accumulate) o += dst[j];
                dst[j] = o;
              }
            }
          }
        }
      }
    }
    if constexpr (Cfg::STAGING_BYTES > 0) {
      if (coop && ok && npend > 0) flush_pending();
      // Stores handed to the TMA unit must have been performed before the CTA may go.
      if (tma_store && lane == 0) {
        const bool arrives = (flags & kFlagPeerSync) != 0 && peer.arrive_flag != nullptr;
        // (shared memory may be given up as soon as the TMA unit has read it; an arrival flag
        // needs the stores themselves to have been performed)
        if ((flags & kFlagEarlyExit) != 0 && !arrives) bulk_wait_read_all();
        else bulk_wait_all();
        if (arrives && ok &&
            *reinterpret_cast<volatile uint32_t*>(status) == kDevOk) {
          // This warp's stores have been performed. Count it; the last warp of the launch tells
          // the other GPU (the fences order every warp's stores, which the counter's chain of
          // atomics has made visible to this one, before the flag). A launch that gave up
          // somewhere raises nothing, so the other side's bounded wait reports it too.
          fence_proxy_async_all();
          __threadfence_system();
          const uint32_t total = gridDim.x * static_cast<uint32_t>(Cfg::EPI_WARPS);
          if (atomicInc(peer.arrive_count, total - 1u) == total - 1u) {
            __threadfence_system();
            st_release_sys(peer.arrive_flag, peer.arrive_value);
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ split warps
    if constexpr (Cfg::REBALANCE) setmaxnreg_dec<Cfg::REGS_XFORM>();
    if constexpr (Cfg::HAS_XFORM) {
      if (warp < Cfg::FIRST_XFORM_WARP + Cfg::XFORM_WARPS) {
        constexpr int XT = Cfg::XFORM_WARPS * 32;
        const int xt = threadIdx.x - Cfg::FIRST_XFORM_WARP * 32;
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        while (ok && sched.next(sg)) {
          for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
            if (!__all_sync(0xffffffffu, mbar_wait(full_bar(s), ph, wc, kDevTimeoutFull))) {
              ok = false;
              break;
            }
            // Element-wise, so the swizzled placement of the raw tile carries over unchanged.
            const uint4* src = reinterpret_cast<const uint4*>(smem_gen + s * Cfg::STAGE_BYTES);
            uint4* dst =
                reinterpret_cast<uint4*>(smem_gen + s * Cfg::STAGE_BYTES + Cfg::RAW_BYTES);
            constexpr int kVecs = Cfg::RAW_BYTES / 16;
            static_assert(kVecs % XT == 0, "whole passes");
#pragma unroll 8
            for (int i = 0; i < kVecs / XT; ++i) {
              const uint4 x = src[i * XT + xt];
              uint4 y;
              y.x = split_small(x.x); y.y = split_small(x.y);
              y.z = split_small(x.z); y.w = split_small(x.w);
              dst[i * XT + xt] = y;
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              if constexpr (CG == 2) mbar_arrive_cluster(ready_bar(s), 0);
              else mbar_arrive(ready_bar(s));
            }
            if (++s == STAGES) { s = 0; ph ^= 1u; }
          }
        }
      }
    }
  }

  // ------------------------------------------------------------ teardown
  __syncwarp();
  // After a failed wait some role left its loop early: give bulk copies still on their way
  // into this CTA's shared memory time to land before the memory is released.
  if (*reinterpret_cast<volatile uint32_t*>(status) != kDevOk) abort_grace_period();
  tcgen05_fence_before_sync();
  if constexpr (CG == 2) cluster_sync(); else __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after_sync();
    tmem_dealloc<CG>(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace rb200
