// roller_b200_gemm_static_scratch: one GEMM entry point that allocates nothing.
//
// Who needs it: a caller that has handed every byte of device memory to its own pool (a
// serving process whose allocator reserved the whole HBM up front has nothing left for a
// library-side cudaMalloc to find), or one that sits in a latency-critical loop, where
// cudaMalloc/cudaFree stall the device because they synchronise it implicitly. The plan-based
// path allocates a status word, events and -- for operands whose rows are not 16-byte aligned --
// padded staging copies of A and B; this entry point does the same work with all of that
// scratch living in a fixed array inside the library image.
//
// Cost and limits: the array occupies kScratchBytes (32 MiB) on every GPU that loads the
// library, from load until the process exits. Staging copies larger than that are refused
// with ROLLER_ERR_TOO_LARGE. Every call uses the same array and leaves its last contents
// there; two calls whose GPU work overlaps (different streams, or different host threads)
// race on it. Nothing in the array has to start at zero except the status word, which each
// call clears on its stream before launching.
//
// Where the memory really comes from: with CUDA's default lazy module loading the array and
// the kernel images get their device memory when they are first touched (the symbol lookup,
// the first launch of each rTile/mode), not when the library is loaded. A caller whose pool
// is about to take all of the device's memory should therefore make one call per rTile and
// mode it will use before the pool does so (or run with CUDA_MODULE_LOADING=EAGER); once that
// is done no later call needs memory from anyone.
#include "../../include/roller_b200.h"

#include <cstdio>
#include <cstring>
#include <mutex>

#include "gemm_launch.h"

namespace {

using namespace rb200;

constexpr size_t kScratchBytes = 32u << 20;
constexpr size_t kScratchFloats = kScratchBytes / sizeof(float);
constexpr int kMaxDevices = 64;

// Staging area for the padded operand copies. In host code this name is only a handle for
// cudaGetSymbolAddress; the device address is resolved once per device below.
static __device__ __align__(256) float g_static_scratch[kScratchFloats];
static __device__ __align__(256) uint32_t g_static_status[64];

constexpr int kMaxVariants = 64;

struct DeviceSetup {
  bool ready = false;
  int max_pairs[kMaxVariants] = {};   // co-resident CTA pairs per cta_group-2 kernel; 0 = not asked yet
  float* scratch = nullptr;     // device address of g_static_scratch on this device
  uint32_t* status = nullptr;   // device address of g_static_status on this device
  int sm_count = 0;
  int cc_major = 0;
  int smem_optin = 0;
};

DeviceSetup g_setup[kMaxDevices];
std::mutex g_setup_mutex;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

bool encode(CUtensorMap* tm, const float* base, long long rows, long long cols, long long ld,
            int box_cols, int box_rows, CUtensorMapSwizzle swz, bool round_to_tf32) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * sizeof(float)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  return fn(tm, round_to_tf32 ? CU_TENSOR_MAP_DATA_TYPE_TFLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box,
            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The staging kernel of this entry point: same copy as the plan path's, writing into the
// library's static array (the destination pointer is the resolved device address).
__global__ void pad_rows_static_kernel(const float* __restrict__ src, long long ld_src,
                                       float* __restrict__ dst, long long ld_dst, int rows,
                                       int cols) {
  const long long total = static_cast<long long>(rows) * cols;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / cols;
    const long long c = i - r * cols;
    dst[r * ld_dst + c] = src[r * ld_src + c];
  }
}

size_t round_up(size_t x, size_t m) { return (x + m - 1) / m * m; }

// One-time set-up for the current device: resolve the device addresses of the static arrays.
int setup_current_device(DeviceSetup** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return ROLLER_ERR_CUDA;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  DeviceSetup& s = g_setup[dev];
  if (!s.ready) {
    void* scratch = nullptr;
    void* status = nullptr;
    if (cudaGetSymbolAddress(&scratch, g_static_scratch) != cudaSuccess) return ROLLER_ERR_CUDA;
    if (cudaGetSymbolAddress(&status, g_static_status) != cudaSuccess) return ROLLER_ERR_CUDA;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return ROLLER_ERR_CUDA;
    s.scratch = static_cast<float*>(scratch);
    s.status = static_cast<uint32_t*>(status);
    s.sm_count = prop.multiProcessorCount;
    s.cc_major = prop.major;
    s.smem_optin = static_cast<int>(prop.sharedMemPerBlockOptin);
    s.ready = true;
  }
  *out = &s;
  return ROLLER_OK;
}

}  // namespace

extern "C" int roller_b200_gemm_static_scratch(const roller_ktile* tile, int mode, int M, int N,
                                               int K, int lda, int ldb, int ldc, const float* A,
                                               const float* B, float* C, uint32_t* dev_status,
                                               void* stream) {
  if (!tile || !A || !B || !C) return ROLLER_ERR_INVALID;
  if (M <= 0 || N <= 0 || K <= 0 || lda < K || ldb < N || ldc < N) return ROLLER_ERR_INVALID;
  if (mode != ROLLER_MODE_1XTF32 && mode != ROLLER_MODE_3XTF32) return ROLLER_ERR_INVALID;
  const KernelVariant* kv =
      find_variant(tile->block_m, tile->block_n, tile->rstep, tile->cta_group, mode, 0);
  if (tile->layout != 0) return ROLLER_ERR_UNSUPPORTED;
  if (!kv) return ROLLER_ERR_UNSUPPORTED;

  DeviceSetup* dev = nullptr;
  int rc = setup_current_device(&dev);
  if (rc != ROLLER_OK) return rc;
  if (dev->cc_major != 10 || dev->smem_optin < kv->smem_bytes) return ROLLER_ERR_DEVICE;
  int variant_idx = -1;
  for (int i = 0; i < variant_count() && i < kMaxVariants; ++i)
    if (&variant_at(i) == kv) variant_idx = i;

  // Which operands break TMA's 16-byte rules and how much of the static array they need.
  const bool stage_a = (lda % 4) != 0 || (reinterpret_cast<uintptr_t>(A) & 15) != 0;
  const bool stage_b = (ldb % 4) != 0 || (reinterpret_cast<uintptr_t>(B) & 15) != 0;
  const size_t pad_lda = round_up(static_cast<size_t>(K), 4);
  const size_t pad_ldb = round_up(static_cast<size_t>(N), 4);
  const size_t a_floats = stage_a ? round_up(pad_lda * static_cast<size_t>(M), 64) : 0;
  const size_t b_floats = stage_b ? round_up(pad_ldb * static_cast<size_t>(K), 64) : 0;
  if (a_floats + b_floats > kScratchFloats) return ROLLER_ERR_TOO_LARGE;

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaFuncSetAttribute(kv->func, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kv->smem_bytes) != cudaSuccess)
    return ROLLER_ERR_CUDA;

  uint32_t* status = dev_status ? dev_status : dev->status;
  if (cudaMemsetAsync(status, 0, sizeof(uint32_t), st) != cudaSuccess) return ROLLER_ERR_CUDA;

  const float* a_src = A;
  const float* b_src = B;
  long long a_ld = lda, b_ld = ldb;
  if (stage_a) {
    float* dst = dev->scratch;
    pad_rows_static_kernel<<<dev->sm_count * 8, 256, 0, st>>>(A, lda, dst,
                                                              static_cast<long long>(pad_lda), M, K);
    a_src = dst;
    a_ld = static_cast<long long>(pad_lda);
  }
  if (stage_b) {
    float* dst = dev->scratch + a_floats;
    pad_rows_static_kernel<<<dev->sm_count * 8, 256, 0, st>>>(B, ldb, dst,
                                                              static_cast<long long>(pad_ldb), K, N);
    b_src = dst;
    b_ld = static_cast<long long>(pad_ldb);
  }
  if ((stage_a || stage_b) && cudaGetLastError() != cudaSuccess) return ROLLER_ERR_CUDA;

  GemmArgs args;
  const bool rnd = (mode == ROLLER_MODE_1XTF32);  // 1xTF32 operands are rounded by the TMA unit
  if (!encode(&args.tmA, a_src, M, K, a_ld, 32, 128, CU_TENSOR_MAP_SWIZZLE_128B, rnd) ||
      !encode(&args.tmB, b_src, K, N, b_ld, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, rnd))
    return ROLLER_ERR_CUDA;
  memset(&args.tmC, 0, sizeof(args.tmC));
  args.C = C;
  args.M = M; args.N = N; args.K = K;
  args.ldc = ldc;
  args.tiles_m = (M + kv->block_m - 1) / kv->block_m;
  args.tiles_n = (N + kv->block_n - 1) / kv->block_n;
  const int num_kb = (K + kv->rstep - 1) / kv->rstep;
  args.chunk_kb = (mode == ROLLER_MODE_3XTF32) ? 4 : num_kb;
  args.acc_kb = args.chunk_kb;
  args.flags = 0;
  if ((ldc % 4) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0) args.flags |= kFlagVecStore;
  args.status = status;
  args.spin_limit = kSpinLimitCycles;
  args.serialize_programmatically = false;
  args.sk_tiles = 0;  // whole tiles only: the stream-K schedule needs a scratch area per CTA
  args.sk_rounds = 1;
  args.sk_ws = nullptr;
  args.sk_flags = nullptr;
  args.epoch = 1;
  args.peer = PeerSync{};
  args.round_plan = RoundPlan{};
  const long long tiles = static_cast<long long>(args.tiles_m) * args.tiles_n;
  int workers = dev->sm_count / kv->cta_group;
  if (kv->cta_group == 2 && variant_idx >= 0) {
    // Same cap as the plan path: no more CTA pairs than the device can hold at once. The
    // occupancy query runs on the host and allocates nothing; its answer is kept per device.
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    int& cached = dev->max_pairs[variant_idx];
    if (cached == 0) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(static_cast<unsigned>(dev->sm_count), 1, 1);
      cfg.blockDim = dim3(static_cast<unsigned>(kv->threads), 1, 1);
      cfg.dynamicSmemBytes = static_cast<size_t>(kv->smem_bytes);
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 2;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kv->func, &cfg) == cudaSuccess && n > 0) cached = n;
      else { cudaGetLastError(); cached = -1; }
    }
    if (cached > 0 && workers > cached) workers = cached;
  }
  const int grid = static_cast<int>(tiles < workers ? tiles : workers) * kv->cta_group;
  if (kv->launch(args, grid, st) != cudaSuccess) {
    cudaGetLastError();
    return ROLLER_ERR_CUDA;
  }
  return ROLLER_OK;
}
