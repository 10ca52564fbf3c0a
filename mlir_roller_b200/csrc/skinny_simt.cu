// fp32 GEMM for a C with very few rows (M <= 16 per pass), on the CUDA cores.
//
// A product like 16 x 8192 x 8192 reads B once (268 MB) and does 2 flop per byte: it is bound by
// HBM, not by arithmetic. The tensor-core kernels serve it well in 1xTF32 (49 us, 0.83 of the
// measured HBM rate), but fp32-level accuracy costs them three MMAs per k-step, and MMAs only 32
// columns wide run far below the tensor rate: 82 us. Plain fp32 FMAs need no split at all, and
// they are exactly the arithmetic of the reference's generated kernel (an fp32 FMA chain per
// output, src/roller.py:280-282). This kernel is that alternative as one more rTile for the
// search to rank. Measured on B200: 86 us for 16 x 8192 x 8192. The profiler shows it bound by
// instruction issue: 80 % of the schedulers' cycles issue, the FMA pipe is busy 53 % (loads from
// the ring, broadcast reads of A, copy bookkeeping and addressing take the rest; Blackwell's
// packed fma.rn.f32x2 was tried to halve the FMA instructions and ran slower, 103 us). So the
// tensor-core skinny tile stays ahead there by 5 %; this one wins where that tile pays for
// staging copies -- it loads with plain
// instructions and takes any alignment (16 x 2049 x 8193: 33 us against 63 us) -- and at
// 16 x 16384 x 16384 (285 against 296 us).
//
// Work split. A CTA owns a strip of 256 columns of C and one range of K; its 8 warps take
// interleaved rows k of that range. Lane l holds the 16 x 8 block of partial sums for columns
// 4l..4l+3 and 128+4l..128+4l+3: per k it takes 32 bytes of B (a warp reads two runs of 512
// contiguous bytes), reads A[0..15][k] from shared memory (four broadcast 128-bit loads) and
// issues 128 FMAs. B arrives through a ring of asynchronous copies (cp.async, 16 rows in flight
// per warp, 128 KB per SM), so the HBM latency is covered by the ring and not by registers. The
// warps' partial blocks are added in warp order (fixed order: results are reproducible bit for
// bit), and the strip's partial tile goes to a workspace [split][M][N]; a second small kernel
// adds the K splits in order and writes C. With one split the first kernel writes C itself.
#include "gemm_launch.h"

namespace rb200 {

namespace {

constexpr int kRows = 16;          // rows of C per pass
constexpr int kStrip = 256;        // columns of C per CTA
constexpr int kCols = kStrip / 32;  // columns per lane (two 128-bit pieces)
constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kChunk = 512;        // k per shared-memory chunk of A (32 KB)
constexpr int kStages = 16;        // rows of B each warp keeps in flight (512 bytes each)
constexpr int kRingBytes = kWarps * kStages * kStrip * 4;   // dynamic shared memory: 64 KB

struct SkinnyArgs {
  const float* A;
  const float* B;
  float* out;            // C, or the workspace [splits][16 * row_groups][N] when splits > 1
  long long lda, ldb, ld_out;
  long long split_stride;  // floats between two splits' partial results in the workspace
  int M, N, K;
  int k_per_split;       // multiple of kChunk
  int vec_b;             // rows of B are 16-byte aligned: 128-bit copies
};

// Asynchronous copy of this lane's four columns of one row of B into its ring slot; columns
// beyond N (and a whole row when `live` is false) arrive as zeros. Bypasses L1: B is streamed.
__device__ __forceinline__ void fetch_b(uint32_t dst, const float* src, int n, int N, bool live,
                                        bool vec) {
  const int cols = live ? max(0, min(4, N - n)) : 0;
  if (vec) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(cols * 4)
                 : "memory");
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst + 4u * j),
                   "l"(src + (j < cols ? j : 0)), "r"(j < cols ? 4 : 0)
                   : "memory");
  }
}
__device__ __forceinline__ void fetch_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void fetch_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
skinny_fp32_kernel(SkinnyArgs a) {
  // A chunk, transposed and in groups of four rows: As[m / 4][k] holds A[m0 + 4 (m / 4) .. + 3][k],
  // so that the four broadcast reads of one k are aligned 128-bit loads
  __shared__ float4 As[kRows / 4][kChunk];
  // Landing ring for B: every warp owns kStages slots of one strip row (128 floats) each; a
  // lane only ever reads the 16 bytes it fetched itself, so the ring needs no barrier.
  extern __shared__ __align__(16) float ring_all[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* ring = ring_all + warp * (kStages * kStrip) + lane * 4;   // second piece: + 128 floats
  const uint32_t ring_s = static_cast<uint32_t>(__cvta_generic_to_shared(ring));
  const int n0 = blockIdx.x * kStrip + lane * 4;        // second piece of columns: n0 + 128
  const int split = blockIdx.y;
  const int m0 = blockIdx.z * kRows;
  const int rows = min(kRows, a.M - m0);
  const int k_begin = split * a.k_per_split;
  const int k_end = min(a.K, k_begin + a.k_per_split);
  const bool vec = a.vec_b != 0;
  // a lane whose columns lie beyond N fetches nothing but zeros, from a valid address
  const float* col = a.B + (n0 < a.N ? n0 : 0);
  const float* col2 = a.B + (n0 + 128 < a.N ? n0 + 128 : 0);

  float acc[kRows][kCols];
#pragma unroll
  for (int m = 0; m < kRows; ++m)
#pragma unroll
    for (int j = 0; j < kCols; ++j) acc[m][j] = 0.f;

  for (int kc = k_begin; kc < k_end; kc += kChunk) {
    const int kn = min(kChunk, k_end - kc);
    // this warp's rows of the chunk: k = warp, warp + 8, ...
    const int nr = kn > warp ? (kn - warp + kWarps - 1) / kWarps : 0;
    const float* bp = col + static_cast<long long>(kc + warp) * a.ldb;
    const float* bp2 = col2 + static_cast<long long>(kc + warp) * a.ldb;
    __syncthreads();   // the previous chunk of A has been consumed
    // A[m0 .. m0+rows)[kc .. kc+kn) -> As, element by element with asynchronous copies (all in
    // flight at once: one round trip to L2 per chunk); rows beyond M and k beyond the range
    // arrive as zeros. This is the oldest copy group, the ring's groups follow it.
    {
      const uint32_t as_s = static_cast<uint32_t>(__cvta_generic_to_shared(&As[0][0]));
      for (int i = threadIdx.x; i < kChunk * kRows; i += kThreads) {
        const int m = i / kChunk, k = i - m * kChunk;     // consecutive threads: consecutive k
        const bool live = m < rows && k < kn;
        const float* src = a.A + (live ? static_cast<long long>(m0 + m) * a.lda + kc + k : 0);
        const uint32_t dst = as_s + ((static_cast<uint32_t>(m >> 2) * kChunk + k) * 4 + (m & 3)) * 4;
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src),
                     "r"(live ? 4 : 0)
                     : "memory");
      }
      fetch_commit();
    }
#pragma unroll
    for (int s = 0; s < kStages; ++s) {
      fetch_b(ring_s + s * (kStrip * 4), bp + static_cast<long long>(s) * kWarps * a.ldb, n0, a.N,
              s < nr, vec);
      fetch_b(ring_s + s * (kStrip * 4) + 512, bp2 + static_cast<long long>(s) * kWarps * a.ldb,
              n0 + 128, a.N, s < nr, vec);
      fetch_commit();
    }
    fetch_wait<kStages>();   // this thread's part of the A chunk has landed ...
    __syncthreads();         // ... and so has everybody else's
    for (int r = 0; r < nr; ++r) {
      fetch_wait<kStages - 1>();     // row r has landed (groups complete in order)
      const int slot = r % kStages;
      const float4 b = *reinterpret_cast<const float4*>(ring + slot * kStrip);
      const float4 b2 = *reinterpret_cast<const float4*>(ring + slot * kStrip + 128);
      const int kk = warp + r * kWarps;
#pragma unroll
      for (int q = 0; q < kRows / 4; ++q) {
        const float4 av = As[q][kk];
        const float am[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          acc[4 * q + t][0] = fmaf(am[t], b.x, acc[4 * q + t][0]);
          acc[4 * q + t][1] = fmaf(am[t], b.y, acc[4 * q + t][1]);
          acc[4 * q + t][2] = fmaf(am[t], b.z, acc[4 * q + t][2]);
          acc[4 * q + t][3] = fmaf(am[t], b.w, acc[4 * q + t][3]);
          acc[4 * q + t][4] = fmaf(am[t], b2.x, acc[4 * q + t][4]);
          acc[4 * q + t][5] = fmaf(am[t], b2.y, acc[4 * q + t][5]);
          acc[4 * q + t][6] = fmaf(am[t], b2.z, acc[4 * q + t][6]);
          acc[4 * q + t][7] = fmaf(am[t], b2.w, acc[4 * q + t][7]);
        }
      }
      // the slot is free again: fetch the row kStages further on into it
      const int rn = r + kStages;
      fetch_b(ring_s + slot * (kStrip * 4), bp + static_cast<long long>(rn) * kWarps * a.ldb, n0,
              a.N, rn < nr, vec);
      fetch_b(ring_s + slot * (kStrip * 4) + 512, bp2 + static_cast<long long>(rn) * kWarps * a.ldb,
              n0 + 128, a.N, rn < nr, vec);
      fetch_commit();
    }
    fetch_wait<0>();   // (only empty groups are left)
  }

  // Add the eight warps' blocks in warp order through shared memory (reusing the A chunk:
  // 16 x 256 floats = 16 KB), then write the strip's tile.
  __syncthreads();
  float* tile = reinterpret_cast<float*>(&As[0][0]);   // [16][128]
  for (int w = 0; w < kWarps; ++w) {
    if (warp == w) {
#pragma unroll
      for (int m = 0; m < kRows; ++m) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float4* t = reinterpret_cast<float4*>(tile + m * kStrip + h * 128 + lane * 4);
          float4 v = make_float4(acc[m][4 * h], acc[m][4 * h + 1], acc[m][4 * h + 2], acc[m][4 * h + 3]);
          if (w > 0) {
            const float4 o = *t;
            v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
          }
          *t = v;
        }
      }
    }
    __syncthreads();
  }
  float* out = a.out + static_cast<long long>(split) * a.split_stride;
  for (int i = threadIdx.x; i < kRows * kStrip; i += kThreads) {
    const int m = i / kStrip, c = i - m * kStrip;
    const int n = blockIdx.x * kStrip + c;
    if (m < rows && n < a.N) out[static_cast<long long>(m0 + m) * a.ld_out + n] = tile[i];
  }
}

// C[m][n] = sum over splits, in split order, of the partial results.
__global__ void skinny_reduce_kernel(const float* __restrict__ ws, long long split_stride,
                                     int splits, float* __restrict__ C, long long ldc, int M, int N) {
  const long long total = static_cast<long long>(M) * N;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int m = static_cast<int>(i / N);
    const int n = static_cast<int>(i - static_cast<long long>(m) * N);
    float s = 0.f;
    for (int p = 0; p < splits; ++p) s += ws[p * split_stride + i];
    C[static_cast<long long>(m) * ldc + n] = s;
  }
}

}  // namespace

const KernelVariant* simt_skinny_variant() {
  static const KernelVariant v = [] {
    KernelVariant k = {};
    k.block_m = kRows;
    k.block_n = kStrip;
    k.rstep = 32;
    k.cta_group = 1;
    k.mode = 3;          // fp32-level accuracy (it is plain fp32 arithmetic)
    k.layout = 3;
    k.stages = 1;
    k.smem_bytes = static_cast<int>(sizeof(float4) * (kRows / 4) * kChunk) + kRingBytes;
    k.tmem_cols = 0;
    k.threads = kThreads;
    k.staging_bytes = 0;
    k.gave_up_stage = 0;
    k.func = reinterpret_cast<const void*>(&skinny_fp32_kernel);
    k.launch = nullptr;  // launched through skinny_simt_launch
    return k;
  }();
  return &v;
}

int skinny_simt_tiles(int M, int N, int* row_groups, int* strips) {
  *row_groups = (M + kRows - 1) / kRows;
  *strips = (N + kStrip - 1) / kStrip;
  return *row_groups * *strips;
}

int skinny_simt_splits(int M, int N, int K, int sm_count) {
  // One CTA per SM at a time. Among the ways to cut K into ranges of whole 512-k chunks, take
  // the one with the shortest schedule: CTAs fill whole waves as evenly as possible, and every
  // split costs one more partial tile written and read (32 / K of the bytes of B each).
  int rg, st;
  const int tiles = skinny_simt_tiles(M, N, &rg, &st);
  const int chunks = (K + kChunk - 1) / kChunk;
  int best = 1;
  double best_cost = 1e30;
  for (int per = 1; per <= chunks; ++per) {
    const int splits = (chunks + per - 1) / per;
    const double ctas = static_cast<double>(tiles) * splits;
    const double waves = ctas / sm_count;
    const double rounds = static_cast<double>((static_cast<long long>(ctas) + sm_count - 1) / sm_count);
    const double cost = rounds / waves * (1.0 + splits * 32.0 / (K > 0 ? K : 1)) +
                        (ctas < sm_count ? 1.0 : 0.0);   // an underfilled machine last
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best = splits;
    }
  }
  return best;
}

size_t skinny_simt_workspace_floats(int M, int N, int splits) {
  return splits > 1 ? static_cast<size_t>(splits) * M * N : 0;
}

cudaError_t skinny_simt_launch(const float* A, const float* B, float* C, int M, int N, int K,
                               long long lda, long long ldb, long long ldc, int splits,
                               float* workspace, int sm_count, cudaStream_t stream) {
  int rg, st;
  skinny_simt_tiles(M, N, &rg, &st);
  const int chunks = (K + kChunk - 1) / kChunk;
  const int chunks_per_split = (chunks + splits - 1) / splits;
  SkinnyArgs a;
  a.A = A; a.B = B;
  a.lda = lda; a.ldb = ldb;
  a.M = M; a.N = N; a.K = K;
  a.k_per_split = chunks_per_split * kChunk;
  a.vec_b = ((reinterpret_cast<uintptr_t>(B) & 15) == 0 && ldb % 4 == 0) ? 1 : 0;
  if (splits > 1) {
    a.out = workspace;
    a.ld_out = N;
    a.split_stride = static_cast<long long>(M) * N;
  } else {
    a.out = C;
    a.ld_out = ldc;
    a.split_stride = 0;
  }
  const dim3 grid(static_cast<unsigned>(st), static_cast<unsigned>(splits), static_cast<unsigned>(rg));
  cudaError_t e = cudaFuncSetAttribute(skinny_fp32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kRingBytes);
  if (e != cudaSuccess) return e;
  skinny_fp32_kernel<<<grid, kThreads, kRingBytes, stream>>>(a);
  e = cudaGetLastError();
  if (e != cudaSuccess || splits == 1) return e;
  const long long total = static_cast<long long>(M) * N;
  int blocks = static_cast<int>((total + 255) / 256);
  if (blocks > sm_count * 8) blocks = sm_count * 8;
  skinny_reduce_kernel<<<blocks, 256, 0, stream>>>(workspace, static_cast<long long>(M) * N, splits,
                                                  C, ldc, M, N);
  return cudaGetLastError();
}

}  // namespace rb200
